"""Learning-rate schedules.

Every schedule here is the product of a linear warm-up ramp and one "shape after warm-up", so the module is built from
those two pieces instead of one class body per schedule: ``Schedule`` owns the optimizer plumbing and the step counter,
and a subclass only says what happens after the ramp (``after_warmup``). The three production schedules
(AF3 staircase, cosine / linear / 1-sqrt anneal, warm-up-stable-decay windows) behave as the reference's
(training/scheduler.py:30-205) and store the same ``last_epoch`` key as ``torch.optim.lr_scheduler.LambdaLR``, so
checkpoints interchange.
"""

from __future__ import annotations

import math
from collections.abc import Callable

# progress in [0, 1] -> remaining fraction in [1, 0]
ANNEAL_CURVES: dict[str, Callable[[float], float]] = {
    "cosine": lambda u: 0.5 + 0.5 * math.cos(math.pi * u),
    "linear": lambda u: 1.0 - u,
    "1-sqrt": lambda u: 1.0 - u**0.5,
}
DECAY_SHAPES = ANNEAL_CURVES  # the name the configuration code looks up


class Schedule:
    """``lr_group = base_lr_group * multiplier(step)``; ``step()`` advances by one optimizer step."""

    warmup_steps: int = 0

    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.base_lrs = [group.get("initial_lr", group["lr"]) for group in optimizer.param_groups]
        self.last_epoch = 0
        self._apply()

    # -- the schedule itself
    def after_warmup(self, step: int) -> float:
        return 1.0

    def multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return step / max(self.warmup_steps, 1)
        return self.after_warmup(step)

    # -- plumbing
    def _apply(self) -> None:
        factor = self.multiplier(self.last_epoch)
        for group, base in zip(self.optimizer.param_groups, self.base_lrs):
            group["lr"] = factor * base

    def step(self) -> None:
        self.last_epoch += 1
        self._apply()

    def get_last_lr(self) -> list[float]:
        return [group["lr"] for group in self.optimizer.param_groups]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch, "_step_count": self.last_epoch + 1, "base_lrs": list(self.base_lrs)}

    def load_state_dict(self, state: dict) -> None:
        self.last_epoch = int(state.get("last_epoch", 0))
        saved = state.get("base_lrs")
        if saved is not None and len(saved) == len(self.base_lrs):
            self.base_lrs = list(saved)
        self._apply()


class ConstantSchedule(Schedule):
    """No schedule (the schedule-free optimizer carries its own warm-up)."""


class AF3LRScheduler(Schedule):
    """AlphaFold-3 staircase: ramp to the peak, hold it until ``start_decay_after``, then multiply by ``decay_factor``
    once per ``decay_every`` steps."""

    def __init__(self, optimizer, cfg):
        self.warmup_steps = int(cfg.warmup_steps)
        self.hold_until, self.every, self.factor = int(cfg.start_decay_after), max(int(cfg.decay_every), 1), float(cfg.decay_factor)
        super().__init__(optimizer)

    def after_warmup(self, step: int) -> float:
        drops = 0 if step < self.hold_until else (step - self.hold_until) // self.every
        return self.factor**drops


class CosineAnnealingScheduler(Schedule):
    """Ramp, optional hold until ``finetune_decay_start``, then one anneal (cosine, linear or 1-sqrt curve) from the peak
    down to ``min_ratio`` of it, reached at ``max_steps`` and kept afterwards."""

    def __init__(self, optimizer, cfg):
        self.warmup_steps = int(cfg.warmup_steps)
        self.curve = ANNEAL_CURVES.get(cfg.finetune_scheduler, ANNEAL_CURVES["cosine"])
        self.anneal_from = max(self.warmup_steps, int(cfg.finetune_decay_start))
        self.max_steps, self.min_ratio = int(cfg.effective_finetune_max_steps), float(cfg.effective_finetune_min_lr_ratio)
        if self.max_steps <= self.anneal_from:
            raise ValueError(f"the anneal would end (finetune_max_steps={self.max_steps}) before it starts (step {self.anneal_from})")
        if self.min_ratio < 0.0 or self.min_ratio > 1.0:
            raise ValueError(f"finetune_min_lr_ratio={self.min_ratio} is not a fraction of the peak rate")
        super().__init__(optimizer)

    def after_warmup(self, step: int) -> float:
        u = (step - self.anneal_from) / (self.max_steps - self.anneal_from)
        u = 0.0 if u < 0.0 else (1.0 if u > 1.0 else u)
        return self.min_ratio + (1.0 - self.min_ratio) * self.curve(u)


class WSDSScheduler(Schedule):
    """Warm-up, stable, decay, and again: inside each ``[start, end)`` window the rate falls from the peak to
    ``min_ratio`` of it along ``1 / (u / min_ratio + 1 - u)`` (harmonic interpolation, fast at first), and jumps back to
    the peak at the window's end. Windows must be well-formed and disjoint."""

    def __init__(self, optimizer, cfg):
        self.warmup_steps = int(cfg.warmup_steps)
        self.min_ratio = float(cfg.wsds_min_lr_ratio)
        if self.min_ratio < 0.0 or self.min_ratio > 1.0:
            raise ValueError(f"wsds_min_lr_ratio={self.min_ratio} is not a fraction of the peak rate")
        self.windows = sorted((int(a), int(b)) for a, b in cfg.wsds_decay_windows)
        previous_end = None
        for a, b in self.windows:
            if b <= a:
                raise ValueError(f"decay window [{a}, {b}) is empty or reversed")
            if previous_end is not None and a < previous_end:
                raise ValueError(f"decay window [{a}, {b}) starts before the previous one ends at {previous_end}")
            previous_end = b
        super().__init__(optimizer)

    def after_warmup(self, step: int) -> float:
        window = next(((a, b) for a, b in self.windows if a <= step < b), None)
        if window is None:
            return 1.0
        u = (step - window[0]) / (window[1] - window[0])
        return 1.0 / (u / max(self.min_ratio, 1e-8) + 1.0 - u)


def build_scheduler(optimizer, cfg) -> Schedule:
    """The schedule ``cfg`` asks for: schedule-free runs get none; otherwise ``finetune_scheduler`` picks it."""
    if cfg.optimizer_type == "schedule_free":
        return ConstantSchedule(optimizer)
    kind = cfg.finetune_scheduler
    table = {"af3": AF3LRScheduler, "wsds": WSDSScheduler, **{name: CosineAnnealingScheduler for name in ANNEAL_CURVES}}
    if kind not in table:
        raise ValueError(f"unknown finetune_scheduler {kind!r}; choose one of {', '.join(sorted(table))}")
    return table[kind](optimizer, cfg)
