"""fp32 islands inside a bf16 autocast region (reference: model/precision.py:23-70)."""

from __future__ import annotations

import functools
from contextlib import nullcontext

import torch


def upcast_fp32(x):
    """Float tensors (also inside dicts / lists / tuples) → fp32; everything else unchanged."""
    if isinstance(x, torch.Tensor):
        return x.float() if x.is_floating_point() else x
    if isinstance(x, dict):
        return {k: upcast_fp32(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return type(x)(upcast_fp32(v) for v in x)
    return x


def _no_autocast(device_type: str = "cuda"):
    return torch.autocast(device_type=device_type, enabled=False)


def fp32_scope(enabled: bool, device_type: str = "cuda"):
    """Context that switches autocast off when ``enabled``; the caller upcasts its own tensors."""
    return _no_autocast(device_type) if enabled else nullcontext()


def fp32_guard(enabled: bool):
    """Decorator: run the call with autocast off and every float argument upcast to fp32."""

    def wrap(fn):
        if not enabled:
            return fn

        @functools.wraps(fn)
        def inner(*args, **kwargs):
            with _no_autocast("cuda"), _no_autocast("cpu"):
                return fn(*(upcast_fp32(a) for a in args), **{k: upcast_fp32(v) for k, v in kwargs.items()})

        return inner

    return wrap
