"""Learning-rate schedules as pure functions of the optimizer step (reference: training/scheduler.py:30-205).

A schedule object exposes ``multiplier(step)``, ``step()``, ``state_dict()`` /
``load_state_dict()`` (``last_epoch`` key, as ``torch.optim.lr_scheduler.LambdaLR``
saves it) and writes ``lr = base_lr * multiplier`` into the optimizer's groups.
"""

from __future__ import annotations

import math

DECAY_SHAPES = {
    "cosine": lambda p: (1.0 + math.cos(math.pi * p)) / 2.0,
    "linear": lambda p: 1.0 - p,
    "1-sqrt": lambda p: 1.0 - math.sqrt(p),
}


class Schedule:
    def __init__(self, optimizer):
        self.optimizer = optimizer
        self.base_lrs = [g.get("initial_lr", g["lr"]) for g in optimizer.param_groups]
        self.last_epoch = 0
        self._apply()

    def multiplier(self, step: int) -> float:  # pragma: no cover - overridden
        return 1.0

    def _apply(self) -> None:
        m = self.multiplier(self.last_epoch)
        for g, base in zip(self.optimizer.param_groups, self.base_lrs):
            g["lr"] = base * m

    def step(self) -> None:
        self.last_epoch += 1
        self._apply()

    def get_last_lr(self) -> list[float]:
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self) -> dict:
        return {"last_epoch": self.last_epoch, "base_lrs": list(self.base_lrs), "_step_count": self.last_epoch + 1}

    def load_state_dict(self, state: dict) -> None:
        self.last_epoch = int(state.get("last_epoch", 0))
        if "base_lrs" in state and len(state["base_lrs"]) == len(self.base_lrs):
            self.base_lrs = list(state["base_lrs"])
        self._apply()


class ConstantSchedule(Schedule):
    pass


class AF3LRScheduler(Schedule):
    """Linear warm-up, plateau, then ``decay_factor`` every ``decay_every`` steps after ``start_decay_after``."""

    def __init__(self, optimizer, cfg):
        self.warmup_steps, self.start_decay_after = cfg.warmup_steps, cfg.start_decay_after
        self.decay_every, self.decay_factor = cfg.decay_every, cfg.decay_factor
        super().__init__(optimizer)

    def multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return step / max(1, self.warmup_steps)
        if step < self.start_decay_after:
            return 1.0
        return self.decay_factor ** ((step - self.start_decay_after) // max(1, self.decay_every))


class CosineAnnealingScheduler(Schedule):
    """Warm-up, optional constant phase, then a cosine / linear / 1-sqrt decay to ``min_ratio``."""

    def __init__(self, optimizer, cfg):
        self.shape = cfg.finetune_scheduler if cfg.finetune_scheduler in DECAY_SHAPES else "cosine"
        self.warmup_steps, self.decay_start = cfg.warmup_steps, cfg.finetune_decay_start
        self.max_steps, self.min_ratio = cfg.effective_finetune_max_steps, cfg.effective_finetune_min_lr_ratio
        start = max(self.warmup_steps, self.decay_start)
        if self.max_steps <= start:
            raise ValueError(f"finetune_max_steps ({self.max_steps}) must be > the decay start ({start})")
        if not 0.0 <= self.min_ratio <= 1.0:
            raise ValueError(f"finetune_min_lr_ratio must be in [0, 1], got {self.min_ratio}")
        super().__init__(optimizer)

    def multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return step / max(1, self.warmup_steps)
        start = max(self.warmup_steps, self.decay_start)
        progress = min(1.0, max(0.0, (step - start) / max(1, self.max_steps - start)))
        return self.min_ratio + (1.0 - self.min_ratio) * DECAY_SHAPES[self.shape](progress)


class WSDSScheduler(Schedule):
    """Warm-up, constant, and inverse-proportional decay inside each ``[start, end)`` window, back to max after it."""

    def __init__(self, optimizer, cfg):
        self.warmup_steps = cfg.warmup_steps
        windows = sorted((int(s), int(e)) for s, e in cfg.wsds_decay_windows)
        for s, e in windows:
            if e <= s:
                raise ValueError(f"wsds_decay_windows: end ({e}) must be > start ({s})")
        for (s1, e1), (s2, e2) in zip(windows[:-1], windows[1:]):
            if s2 < e1:
                raise ValueError(f"wsds_decay_windows overlap: [{s1}, {e1}) and [{s2}, {e2})")
        self.windows, self.min_ratio = windows, float(cfg.wsds_min_lr_ratio)
        if not 0.0 <= self.min_ratio <= 1.0:
            raise ValueError(f"wsds_min_lr_ratio must be in [0, 1], got {self.min_ratio}")
        super().__init__(optimizer)

    def multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return step / max(1, self.warmup_steps)
        for start, end in self.windows:
            if start <= step < end:
                u = (step - start) / (end - start)
                return 1.0 / (u / max(self.min_ratio, 1e-8) + (1.0 - u))
        return 1.0


def build_scheduler(optimizer, cfg) -> Schedule:
    if cfg.optimizer_type == "schedule_free":
        return ConstantSchedule(optimizer)
    name = cfg.finetune_scheduler
    if name in DECAY_SHAPES:
        return CosineAnnealingScheduler(optimizer, cfg)
    if name == "wsds":
        return WSDSScheduler(optimizer, cfg)
    if name == "af3":
        return AF3LRScheduler(optimizer, cfg)
    raise ValueError(f"finetune_scheduler must be 'af3', 'cosine', 'linear', '1-sqrt' or 'wsds'; got {name!r}")
