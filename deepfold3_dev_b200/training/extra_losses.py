"""Optional structure losses: chirality, backbone chirality, FAPE, shape complementarity.

All are off in the default recipe (their ``alpha_*`` weights are 0); reference:
training/loss.py:392-755 (shape complementarity), :1531-1798 (FAPE), :2045-2320 (chirality).
"""

from __future__ import annotations

import torch


def _pending(name: str):
    raise NotImplementedError(f"{name} is not available in this build yet; keep its alpha at 0")


def chirality_loss(*args, **kwargs):
    _pending("chirality_loss")


def chirality_violation_rates(*args, **kwargs):
    _pending("chirality_violation_rates")


def backbone_chirality_loss(*args, **kwargs):
    _pending("backbone_chirality_loss")


def fape_from_features(*args, **kwargs):
    _pending("fape_loss")


def shape_complementarity_loss(*args, **kwargs):
    _pending("shape_complementarity_loss")


def shape_comp_kwargs(cfg) -> dict:
    return {}


def shape_comp_sample_weight(cfg, noise_levels: torch.Tensor):
    return None
