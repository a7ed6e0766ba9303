"""Schedule-free AdamW on the flat buffers (reference: training/schedule_free.py:101-368).

Defazio et al. 2024: the parameters hold ``y = (1 - beta1) z + beta1 x`` while training, ``z`` takes the
AdamW step, ``x`` is the running average ``x <- (1 - c) x + c z`` with ``c = w_k / sum w_i``,
``w_k = k^r * lr_max^p``. With ``decoupling_parameter = C`` the averaging weight becomes
``min(1, (1 - beta1) * C * c)`` (refined schedule-free averaging). ``eval()`` moves the parameters to
``x``, ``train()`` back to ``y``. The whole update is a handful of vector operations on the flat
buffers, one launch each.
"""

from __future__ import annotations

import math

import torch

import contextlib

from .flat_optimizer import FlatAdamW


@contextlib.contextmanager
def optimizer_eval_mode(optimizer):
    """Parameters hold the averaged iterate ``x`` inside the block (schedule-free only; a no-op for AdamW).

    Checkpoints are written and evaluations run under this, as in the reference
    (training/schedule_free.py ``optimizer_eval_mode``, training/checkpointing.py:291).
    """
    flip = isinstance(optimizer, FlatAdamWScheduleFree) and optimizer.train_mode
    if flip:
        optimizer.eval()
    try:
        yield
    finally:
        if flip:
            optimizer.train()


class FlatAdamWScheduleFree(FlatAdamW):
    def __init__(self, model, lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, warmup_steps=0, r=0.0,
                 weight_lr_power=2.0, decoupling_parameter=None, strong_decay=None, ema_decay=0.0):  # fmt: skip
        if decoupling_parameter is not None and decoupling_parameter <= 0:
            raise ValueError(f"decoupling_parameter must be > 0 or None, got {decoupling_parameter}")
        super().__init__(model, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, strong_decay=strong_decay,
                         ema_decay=ema_decay)  # fmt: skip
        self.warmup_steps, self.r, self.weight_lr_power = int(warmup_steps), float(r), float(weight_lr_power)
        self.decoupling_parameter = decoupling_parameter
        self.z = self.flat_param.clone()
        self.exp_avg = None  # schedule-free keeps no first moment
        self.train_mode = True
        self.weight_sum, self.lr_max, self.scheduled_lr = 0.0, -1.0, 0.0

    # ---- mode switches: parameters are y in train mode, x in eval mode
    @torch.no_grad()
    def eval(self) -> None:
        if self.train_mode:
            b1 = self.param_groups[0]["betas"][0]
            self.flat_param.lerp_(self.z, 1.0 - 1.0 / b1)
            self.train_mode = False
            self.refresh_bf16()

    @torch.no_grad()
    def train(self) -> None:
        if not self.train_mode:
            b1 = self.param_groups[0]["betas"][0]
            self.flat_param.lerp_(self.z, 1.0 - b1)
            self.train_mode = True
            self.refresh_bf16()

    @torch.no_grad()
    def step(self, grad_scale=1.0, update_ema: bool = True) -> None:
        if not self.train_mode:
            raise RuntimeError("schedule-free step() in eval mode: call optimizer.train() first")
        self.step_count += 1
        k = self.step_count
        g0 = self.param_groups[0]
        lr_peak, (b1, b2), eps = g0["lr"], g0["betas"], g0["eps"]
        sched = min(1.0, k / self.warmup_steps) if self.warmup_steps > 0 else 1.0
        bc2 = 1.0 - b2**k
        lr = lr_peak * sched * math.sqrt(bc2)
        self.scheduled_lr = lr
        self.lr_max = max(lr, self.lr_max)
        weight = (k**self.r) * (self.lr_max**self.weight_lr_power)
        self.weight_sum += weight
        c = weight / self.weight_sum if self.weight_sum > 0 else 0.0
        if self.decoupling_parameter is not None:
            c = min(1.0, (1.0 - b1) * self.decoupling_parameter * c)
        g = self.flat_grad * grad_scale
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1.0 - b2)
        gn = g / (self.exp_avg_sq.sqrt().add_(eps))
        gn.add_(self.flat_param * self.decay_vec)
        y = self.flat_param
        y.lerp_(self.z, c)
        y.add_(gn, alpha=lr * (b1 * (1.0 - c) - 1.0))
        self.z.sub_(gn, alpha=lr)
        if update_ema and self.shadow is not None:
            # the shadow follows the averaged iterate x = (y - (1 - b1) z) / b1, as the reference's EMA callback does
            # under optimizer_eval_mode
            self.ema_updates += 1
            x = torch.lerp(self.flat_param, self.z, 1.0 - 1.0 / b1)
            self.shadow.lerp_(x, 1.0 - self.ema_decay)
        self.refresh_bf16()

    @torch.no_grad()
    def reseed_z(self) -> None:
        """``z := parameters``: after a broadcast or a weight load that did not restore the optimizer state."""
        self.z.copy_(self.flat_param)
        self.train_mode = True

    # ---- checkpoint layout: torch-style per-parameter state with z
    def state_dict(self) -> dict:
        state = {}
        if self.step_count > 0:
            for i in range(len(self.params)):
                state[self._torch_index[i]] = {"z": self._view(self.z, i).clone(),
                                               "exp_avg_sq": self._view(self.exp_avg_sq, i).clone()}  # fmt: skip
        groups = [{**{k: v for k, v in g.items() if k != "params"}, "k": self.step_count, "train_mode": self.train_mode,
                   "weight_sum": self.weight_sum, "lr_max": self.lr_max, "scheduled_lr": self.scheduled_lr,
                   "warmup_steps": self.warmup_steps, "r": self.r, "weight_lr_power": self.weight_lr_power,
                   "decoupling_parameter": self.decoupling_parameter, "params": list(g["params"])}
                  for g in self.param_groups]  # fmt: skip
        return {"state": state, "param_groups": groups}

    @torch.no_grad()
    def load_state_dict(self, sd: dict) -> None:
        inv = {k: i for i, k in self._torch_index.items()}
        for k, st in sd.get("state", {}).items():
            i = inv[int(k)]
            self._view(self.z, i).copy_(st["z"])
            self._view(self.exp_avg_sq, i).copy_(st["exp_avg_sq"])
        g = (sd.get("param_groups") or [{}])[0]
        self.step_count = int(g.get("k", 0))
        self.weight_sum, self.lr_max = float(g.get("weight_sum", 0.0)), float(g.get("lr_max", -1.0))
        self.scheduled_lr = float(g.get("scheduled_lr", 0.0))
        # the reference saves under eval mode (parameters = x, train_mode False) and switches back with train()
        # after loading; the caller (CheckpointManager.load) does the same here
        self.train_mode = bool(g.get("train_mode", True))
        for mine, theirs in zip(self.param_groups, sd.get("param_groups", [])):
            for key in ("lr", "initial_lr", "betas", "eps", "weight_decay"):
                if key in theirs:
                    mine[key] = tuple(theirs[key]) if key == "betas" else theirs[key]
