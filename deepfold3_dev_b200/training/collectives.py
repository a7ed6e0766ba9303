"""Picking one example out of a batched feature tree inside the training step (reference: training/collectives.py)."""

from __future__ import annotations

import torch


def slice_batch_dict(tree: dict, index: int, batch_size: int) -> dict:
    """``tree`` with every tensor that carries the batch axis (leading size ``batch_size``) replaced by its entry
    ``index``. Nested dicts are walked; tensors without the batch axis, scalars and strings come back unchanged."""

    def pick(value):
        if isinstance(value, dict):
            return {name: pick(item) for name, item in value.items()}
        batched = isinstance(value, torch.Tensor) and value.dim() > 0 and value.shape[0] == batch_size
        return value[index] if batched else value

    return pick(tree)
