"""Run-local counters and seeding (reference: training/state.py:22-94)."""

from __future__ import annotations

import os
import random
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class TrainState:
    global_step: int = 0  # micro-steps, accumulation included
    effective_step: int = 0  # optimizer steps taken
    epoch: int = 0
    best_eval_loss: float = field(default_factory=lambda: float("inf"))
    consecutive_nan_skips: int = 0
    last_grad_norm: torch.Tensor | None = None
    last_grad_norm_global: torch.Tensor | None = None
    last_grad_norm_rank_mean: torch.Tensor | None = None
    last_grad_norm_rank_max: torch.Tensor | None = None
    last_null_pair_grad_norm: torch.Tensor | None = None
    last_num_recycles: int = 0


def seed_everything(seed: int, rank: int, *, deterministic: bool = False) -> None:
    """Seed python / numpy / torch with ``seed + rank``; optionally force deterministic algorithms."""
    s = seed + rank
    random.seed(s)
    np.random.seed(s)
    torch.manual_seed(s)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(s)
    if deterministic:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)
        torch.backends.cudnn.deterministic = True
        torch.backends.cudnn.benchmark = False
