"""Small pytree helpers used inside the training step (reference: training/collectives.py)."""

from __future__ import annotations

import torch


def slice_batch_dict(d: dict, b: int, batch_size: int) -> dict:
    """Element ``b`` of every tensor whose leading size is ``batch_size``; other values pass through."""
    out = {}
    for k, v in d.items():
        if isinstance(v, torch.Tensor):
            out[k] = v[b] if v.dim() >= 1 and v.shape[0] == batch_size else v
        elif isinstance(v, dict):
            out[k] = slice_batch_dict(v, b, batch_size)
        else:
            out[k] = v
    return out
