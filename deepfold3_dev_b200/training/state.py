"""Counters of a training run and process-wide seeding.

``TrainState`` is what a checkpoint's ``global_step`` / ``effective_step`` / ``epoch`` / ``best_eval_loss`` entries are
read from and restored into (reference: training/state.py:22-94); the remaining fields are the latest gradient-norm
readings that the logging code picks up, kept as device tensors so that recording them never waits for the GPU.
"""

from __future__ import annotations

import dataclasses
import os
import random

import numpy as np
import torch


@dataclasses.dataclass
class TrainState:
    # progress
    global_step: int = 0        # micro-batches seen (gradient accumulation counts each one)
    effective_step: int = 0     # optimizer updates applied
    epoch: int = 0
    best_eval_loss: float = float("inf")
    consecutive_nan_skips: int = 0
    last_num_recycles: int = 0
    # latest gradient statistics
    last_grad_norm: torch.Tensor | None = None
    last_grad_norm_global: torch.Tensor | None = None
    last_grad_norm_rank_mean: torch.Tensor | None = None
    last_grad_norm_rank_max: torch.Tensor | None = None
    last_null_pair_grad_norm: torch.Tensor | None = None


def seed_everything(seed: int, rank: int, *, deterministic: bool = False) -> None:
    """Every generator of this process (python, numpy, torch CPU and CUDA) starts from ``seed + rank``, so ranks draw
    different noise and masks from one configured seed. ``deterministic`` additionally asks torch, cuBLAS and cuDNN for
    reproducible algorithms (slower; warns where none exists)."""
    value = int(seed) + int(rank)
    for seeder in (random.seed, np.random.seed, torch.manual_seed):
        seeder(value)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(value)
    if not deterministic:
        return
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
    torch.backends.cudnn.benchmark = False
    torch.backends.cudnn.deterministic = True
    torch.use_deterministic_algorithms(True, warn_only=True)
