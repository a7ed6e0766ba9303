"""Autograd wrappers around ``torch.ops.df3`` (the sm_100a kernels).

Each ``Function`` saves exactly what its backward kernel reads. Non-contiguous
inputs are made contiguous here, so callers can pass views.
"""

from __future__ import annotations

import collections

import torch

LAUNCHES: collections.Counter = collections.Counter()


class _Ops:
    """``torch.ops.df3`` with a per-kernel launch count (read by the benchmark's ``gpu_launches``)."""

    def __getattr__(self, name):
        op = getattr(torch.ops.df3, name)

        def call(*args, **kwargs):
            LAUNCHES[name] += 1
            return op(*args, **kwargs)

        return call


K = _Ops()


def launch_count(reset: bool = False) -> int:
    n = sum(LAUNCHES.values())
    if reset:
        LAUNCHES.clear()
    return n


def next_mask_seed() -> int:
    """Seed of the next dropout mask, drawn from torch's global CPU generator.

    ``seed_everything`` seeds torch with ``seed + rank``, so ranks draw different
    masks. The global generator (not a private one) is used on purpose:
    activation checkpointing saves and restores its state around the recompute,
    so the recomputed forward regenerates the same mask as the original one.
    """
    return int(torch.randint(0, 2**31 - 1, (1,)).item())


def _f32(t):
    return None if t is None else (t if t.dtype == torch.float32 else t.float())


class _LayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        xc = x.contiguous()
        w, b = _f32(weight), _f32(bias)
        y, mean, rstd = K.layer_norm_fwd(xc, w, b, eps)
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.has_w, ctx.has_b = weight is not None, bias is not None
        ctx.w_dtype = None if weight is None else weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        need_wb = (ctx.has_w and ctx.needs_input_grad[1]) or (ctx.has_b and ctx.needs_input_grad[2])
        dx, partial = K.layer_norm_bwd(dy.contiguous(), x, w, mean, rstd, need_wb)
        dw = db = None
        if need_wb:
            sums = partial.sum(0)
            if ctx.has_w:
                dw = sums[0].to(ctx.w_dtype)
            if ctx.has_b:
                db = sums[1].to(ctx.b_dtype)
        return dx, dw, db, None


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    return _LayerNorm.apply(x, weight, bias, eps)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return K.swiglu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return K.swiglu_bwd(dy.contiguous(), x)


def swiglu(x):
    return _SwiGLU.apply(x)


class _DropoutAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, residual, x, p, share_rows, seed):
        xc = x.contiguous()
        A, B, C = xc.shape[-3], xc.shape[-2], xc.shape[-1]
        ctx.meta = (A, B, C, share_rows, p, seed)
        return K.dropout_shared(residual.contiguous(), xc, A, B, C, share_rows, p, seed)

    @staticmethod
    def backward(ctx, dy):
        A, B, C, share_rows, p, seed = ctx.meta
        dyc = dy.contiguous()
        return dyc, K.dropout_shared(None, dyc, A, B, C, share_rows, p, seed), None, None, None


def dropout_add(residual, x, p: float, share_dim: int, seed: int | None = None):
    """``residual + dropout(x)`` with the draw shared along ``share_dim`` (-3 rows, -2 columns)."""
    if share_dim not in (-3, -2):
        raise ValueError("share_dim must be -3 or -2")
    if seed is None:
        seed = next_mask_seed()
    return _DropoutAdd.apply(residual, x, float(p), share_dim == -3, int(seed))


def adamw_ema_flat(p, g, m, v, ema, decay, scale, lr, b1, b2, eps, bc1, bc2, ema_w):
    K.adamw_ema(p, g, m, v, ema, decay, scale, lr, b1, b2, eps, bc1, bc2, ema_w)
