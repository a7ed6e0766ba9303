"""Autograd wrappers around ``torch.ops.df3`` (the sm_100a kernels).

Each ``Function`` saves exactly what its backward kernel reads. Non-contiguous
inputs are made contiguous here, so callers can pass views.
"""

from __future__ import annotations

import collections
import os
import weakref

import torch

LAUNCHES: collections.Counter = collections.Counter()


NVTX = os.environ.get("DF3_NVTX", "0") == "1"  # one NVTX range per kernel-op call: names the launches in a timeline


class _Ops:
    """``torch.ops.df3`` with a per-kernel launch count (read by the benchmark's ``gpu_launches``) and, with
    ``DF3_NVTX=1``, an NVTX range ``df3::<op>`` around every call."""

    def __getattr__(self, name):
        op = getattr(torch.ops.df3, name)

        def call(*args, **kwargs):
            LAUNCHES[name] += 1
            if not NVTX:
                return op(*args, **kwargs)
            torch.cuda.nvtx.range_push(f"df3::{name}")
            try:
                return op(*args, **kwargs)
            finally:
                torch.cuda.nvtx.range_pop()

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
            dw = sums[0] if ctx.has_w else None
            db = sums[1] if ctx.has_b else None
            if dw is not None and dw.dtype != ctx.w_dtype:
                dw = dw.to(ctx.w_dtype)
            if db is not None and db.dtype != ctx.b_dtype:
                db = db.to(ctx.b_dtype)
        return dx, dw, db, None


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    return _LayerNorm.apply(x, weight, bias, eps)


class _PlaneLayerNorm(torch.autograd.Function):
    """LayerNorm over the channel axis of channel-major ``x [C, M]``, returned channel-last ``[M, C]``."""

    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        xc = x.contiguous()
        w, b = _f32(weight), _f32(bias)
        y, mean, rstd = K.plane_layer_norm_fwd(xc, w, b, eps)
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.has_w, ctx.has_b = weight is not None, bias is not None
        ctx.w_dtype = None if weight is None else weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, mean, rstd = ctx.saved_tensors
        need_wb = (ctx.has_w and ctx.needs_input_grad[1]) or (ctx.has_b and ctx.needs_input_grad[2])
        dyc = dy.contiguous()
        if dyc.dtype != torch.bfloat16:
            dyc = dyc.to(torch.bfloat16)
        dx, partial = K.plane_layer_norm_bwd(dyc, x, w, mean, rstd, need_wb)
        dw = db = None
        if need_wb:
            sums = partial.sum(0)
            dw = sums[0].to(ctx.w_dtype) if ctx.has_w else None
            db = sums[1].to(ctx.b_dtype) if ctx.has_b else None
        return dx, dw, db, None


def plane_layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    return _PlaneLayerNorm.apply(x, weight, bias, eps)


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
        return K.dropout_shared(residual.contiguous(), xc, A, B, C, share_rows, p, seed, None)

    @staticmethod
    def backward(ctx, dy):
        A, B, C, share_rows, p, seed = ctx.meta
        dyc = dy.contiguous()
        return dyc, K.dropout_shared(None, dyc, A, B, C, share_rows, p, seed, None), None, None, None


class _DropoutAddDeviceSeed(torch.autograd.Function):
    """Dropout-add whose mask derives from a device-resident base seed plus a fixed offset: the form a CUDA-graph
    capture can hold. Backward regenerates the mask from the same seed tensor, which the owner of the graph changes
    only before a forward replay."""

    @staticmethod
    def forward(ctx, residual, x, p, share_rows, offset, seed_dev):
        xc = x.contiguous()
        A, B, C = xc.shape[-3], xc.shape[-2], xc.shape[-1]
        ctx.meta = (A, B, C, share_rows, p, offset)
        ctx.seed_dev = seed_dev
        return K.dropout_shared(residual.contiguous(), xc, A, B, C, share_rows, p, offset, seed_dev)

    @staticmethod
    def backward(ctx, dy):
        A, B, C, share_rows, p, offset = ctx.meta
        dyc = dy.contiguous()
        return dyc, K.dropout_shared(None, dyc, A, B, C, share_rows, p, offset, ctx.seed_dev), None, None, None, None


def dropout_add(residual, x, p: float, share_dim: int, seed: int | None = None):
    """``residual + dropout(x)`` with the draw shared along ``share_dim`` (-3 rows, -2 columns)."""
    if share_dim not in (-3, -2):
        raise ValueError("share_dim must be -3 or -2")
    from ..utils.cuda_graph import GraphSeed

    gs = GraphSeed.current
    if gs is not None and seed is None and not torch.is_grad_enabled():
        # inside a region that is captured into a CUDA graph: the base seed lives on the device and is refreshed per replay
        xc = x.contiguous()
        return K.dropout_shared(residual.contiguous(), xc, xc.shape[-3], xc.shape[-2], xc.shape[-1], share_dim == -3, float(p),
                                gs.offset(), gs.tensor)  # fmt: skip
    if gs is not None and seed is None:
        return _DropoutAddDeviceSeed.apply(residual, x, float(p), share_dim == -3, gs.offset(), gs.tensor)
    if seed is None:
        seed = next_mask_seed()
    return _DropoutAdd.apply(residual, x, float(p), share_dim == -3, int(seed))


def adamw_ema_flat(p, g, m, v, ema, decay, scale, lr, b1, b2, eps, bc1, bc2, ema_w, p16=None):
    K.adamw_ema(p, g, m, v, ema, decay, scale, lr, b1, b2, eps, bc1, bc2, ema_w, p16)
    _W16.clear()  # stacked copies were built from the old values


# ------------------------------------------------------------------------------------------------
# tcgen05 GEMM family. Forward runs the fused-epilogue kernel; backward recomputes the pre-activation
# with a library GEMM (nothing of size [rows, 2 * hidden] is kept between forward and backward).
BF16 = torch.bfloat16
_W16: dict = {}  # (data_ptr, shape) per weight -> (versions, bf16 tensor); emptied whenever parameters change


def _cache_put(key, value, sources) -> None:
    """Store a cast and tie its life to the tensors it was made from: when one of them is collected the entry goes too.
    Keys are storage addresses, and the allocator hands a freed parameter's address (with an equal version counter) to
    the next model built in the process; without the eviction that model would be served the old model's weights."""
    if len(_W16) > 50000:
        _W16.clear()
    _W16[key] = value
    for w in sources:
        weakref.finalize(w, _W16.pop, key, None)
_MIRROR: dict = {}  # (data_ptr, shape) of an fp32 parameter -> [bf16 view kept current by the optimizer, version]


def register_bf16_mirror(param, view16) -> None:
    """Tell the cache that ``view16`` always holds ``param`` in bf16 (the flat optimizer refreshes it every step)."""
    _MIRROR[(param.data_ptr(), tuple(param.shape))] = [view16, param._version, weakref.ref(param.untyped_storage())]


def invalidate_weight_cache(clear_mirrors: bool = False) -> None:
    """Drop cached bf16 copies; call after parameters were written in place behind autograd's back."""
    _W16.clear()
    if clear_mirrors:
        _MIRROR.clear()


def _one_bf16(w):
    hit = _MIRROR.get((w.data_ptr(), tuple(w.shape)))
    if hit is not None and w.dtype == torch.float32 and hit[2]() is w.untyped_storage():
        if hit[1] != w._version:  # written directly (load_state_dict, init): refresh this view
            with torch.no_grad():
                hit[0].copy_(w)
            hit[1] = w._version
        return hit[0]
    return None


def bf16_weight(*ws):
    """bf16 copy of one weight, or of several stacked along the rows.

    Parameters owned by the flat optimizer resolve to views of its bf16 mirror (no kernel). Everything else is
    cast once and cached by storage address and version until ``invalidate_weight_cache``. Keys are storage
    addresses, not object identities: activation checkpointing hands the backward detached aliases of the
    parameters.
    """
    if len(ws) == 1:
        m = _one_bf16(ws[0])
        if m is not None:
            return m
    capturing = ws[0].is_cuda and torch.cuda.is_current_stream_capturing()
    key = tuple((w.data_ptr(), tuple(w.shape)) for w in ws)
    sig = tuple(w._version for w in ws)
    hit = None if capturing else _W16.get(key)
    if hit is not None and hit[0] == sig:
        return hit[1]
    with torch.no_grad():
        parts = [_one_bf16(w) for w in ws]
        parts = [p if p is not None else w.detach().to(BF16) for p, w in zip(parts, ws)]
        t = (parts[0] if len(parts) == 1 else torch.cat(parts, 0)).contiguous()
    if not capturing:  # a cast made inside a CUDA-graph capture belongs to that graph's pool
        _cache_put(key, (sig, t), ws)
    return t


def _bf16c(x):
    return x.to(BF16).contiguous()


def _mm_ok(*ts) -> bool:
    """Operands the tcgen05 product takes as they are: bf16 CUDA, every extent a multiple of 8."""
    return all(t.is_cuda and t.dtype == BF16 and t.numel() > 0 and all(d % 8 == 0 for d in t.shape[-2:]) for t in ts)


def mm(a, b, trans_a: bool = False, trans_b: bool = False, out_fp32: bool = False, splits: int = 1, out=None):
    """``op(a) @ op(b)`` (2-D, or 3-D batched) on the tcgen05 kernel; ``trans_*`` hands an operand over transposed
    instead of copying it. Falls back to torch for shapes the kernel does not take (extents not multiples of 8)."""
    if _mm_ok(a, b):
        return K.matmul(a, b, trans_a, trans_b, out_fp32, splits, out)
    if out is None and all(t.is_cuda and t.dtype == BF16 and t.numel() > 0 and t.dim() in (2, 3) for t in (a, b)):
        # a ragged extent (4 attention heads, an odd token count): zero rows / columns up to the next multiple of 8
        # change nothing in the product, so pad the operand that needs it and cut the result back
        def pad8(t):
            r, c = (-t.shape[-2]) % 8, (-t.shape[-1]) % 8
            return torch.nn.functional.pad(t, (0, c, 0, r)) if (r or c) else t

        rows = a.shape[-1] if trans_a else a.shape[-2]
        cols = b.shape[-2] if trans_b else b.shape[-1]
        full = K.matmul(pad8(a), pad8(b), trans_a, trans_b, out_fp32, splits, None)
        return full[..., :rows, :cols] if full.shape[-2:] == (rows, cols) else full[..., :rows, :cols].contiguous()
    A = a.transpose(-1, -2) if trans_a else a
    B = b.transpose(-1, -2) if trans_b else b
    r = torch.matmul(A, B)
    r = r.float() if out_fp32 else r
    if out is not None:
        out.copy_(r.view(out.shape))
        return out
    return r


def _wgrad(dy2d, x2d, like):
    """``dy2d.T @ x2d`` accumulated in fp32 (split along the rows, partial sums added in a fixed order), in the dtype
    of the parameter ``like``."""
    return mm(dy2d, x2d, True, False, True, 0).to(like.dtype)


def _plain_gemm(x16, W, bias=None):
    """``x16 W^T (+ bias)`` with x16 [..., K] bf16 and W [N, K] bf16."""
    if x16.is_cuda and x16.shape[-1] % 8 == 0 and x16.numel() > 0:
        return K.gemm(x16, W, bias, None, None, 0, False)
    y = torch.matmul(x16, W.t())
    return y if bias is None else y + bias.to(y.dtype)


def gemm_supported(x, w) -> bool:
    return x.is_cuda and x.shape[-1] % 8 == 0 and x.shape[-1] >= 16 and x.numel() > 0


def _stacked_gate_proj(w_gate, w_proj, deinterleave: bool):
    """``[w_gate; w_proj]`` in bf16; with ``deinterleave`` each half lists its even rows first, then its odd rows."""
    if not deinterleave:
        return bf16_weight(w_gate, w_proj)
    capturing = w_gate.is_cuda and torch.cuda.is_current_stream_capturing()
    key = ("deint", w_gate.data_ptr(), w_proj.data_ptr(), tuple(w_gate.shape))
    sig = (w_gate._version, w_proj._version)
    hit = None if capturing else _W16.get(key)
    if hit is not None and hit[0] == sig:
        return hit[1]
    with torch.no_grad():
        parts = [w.detach()[i::2] for w in (w_gate, w_proj) for i in (0, 1)]
        t = torch.cat(parts, 0).to(BF16).contiguous()
    if not capturing:
        _cache_put(key, (sig, t), (w_gate, w_proj))
    return t


def _reinterleave(dw_half):
    n = dw_half.shape[0] // 2
    return torch.stack([dw_half[:n], dw_half[n:]], 1).reshape(dw_half.shape)


class _GatedDual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_gate, w_proj, mask, planes, deinterleave):
        x16 = _bf16c(x)
        W = _stacked_gate_proj(w_gate, w_proj, deinterleave)
        m = None if mask is None else mask.reshape(-1).float()
        ctx.save_for_backward(x16, w_gate, w_proj, m)
        ctx.x_dtype, ctx.planes, ctx.deinterleave = x.dtype, planes, deinterleave
        return K.gemm(x16, W, None, m, None, 1, planes)

    @staticmethod
    def backward(ctx, dy):
        x16, w_gate, w_proj, m = ctx.saved_tensors
        W = _stacked_gate_proj(w_gate, w_proj, ctx.deinterleave)
        n = w_gate.shape[0]
        x2 = x16.reshape(-1, x16.shape[-1])
        dy2 = (dy.t() if ctx.planes else dy.reshape(-1, n)).to(BF16).contiguous()
        dgp = K.gemm(x2, W, None, m, dy2, 5, False)  # pre-activations recomputed in the accumulator
        dx = mm(dgp, W).view(x16.shape).to(ctx.x_dtype)
        dW = _wgrad(dgp, x2, w_gate)
        dg, dp = dW[:n], dW[n:]
        if ctx.deinterleave:
            dg, dp = _reinterleave(dg), _reinterleave(dp)
        return dx, dg, dp, None, None, None


def gated_dual_linear(x, w_gate, w_proj, mask=None, planes: bool = False, deinterleave: bool = False):
    """``sigmoid(x w_gate^T) * (x w_proj^T) * mask``.

    ``planes=True`` returns ``[channels, rows]``; ``deinterleave=True`` orders the output channels
    even-first (0, 2, 4, ..., 1, 3, 5, ...), which puts the two operands of the triangle contraction
    into two contiguous halves.
    """
    return _GatedDual.apply(x, w_gate, w_proj, mask, planes, deinterleave)


class _StackedLinear(torch.autograd.Function):
    """``x [w_0; w_1; ...]^T`` as one GEMM on the cached stacked bf16 weight."""

    @staticmethod
    def forward(ctx, x, *ws):
        x16 = _bf16c(x)
        ctx.save_for_backward(x16, *ws)
        ctx.x_dtype = x.dtype
        return _plain_gemm(x16, bf16_weight(*ws))

    @staticmethod
    def backward(ctx, dy):
        x16, *ws = ctx.saved_tensors
        W = bf16_weight(*ws)
        x2 = x16.reshape(-1, x16.shape[-1])
        d = dy.reshape(-1, W.shape[0]).to(BF16)
        dx = mm(d, W).view(x16.shape).to(ctx.x_dtype)
        dW = mm(d, x2, True, False, True, 0)
        outs, r = [], 0
        for w in ws:
            outs.append(dW[r : r + w.shape[0]].to(w.dtype))
            r += w.shape[0]
        return (dx, *outs)


def stacked_linear(x, *ws):
    return _StackedLinear.apply(x, *ws)


def _linear_fwd(x, w, b):
    x16 = x if x.dtype == BF16 else x.to(BF16)
    W = bf16_weight(w)
    if x16.shape[-1] % 8 == 0 and x16.numel() > 0:
        return K.gemm(x16, W, b, None, None, 0, False)  # bias added in fp32 in the epilogue
    if b is None:
        return torch.matmul(x16, W.t())
    return torch.addmm(bf16_weight(b), x16.reshape(-1, x16.shape[-1]), W.t()).view(*x16.shape[:-1], W.shape[0])


class _Linear(torch.autograd.Function):
    """``x w^T + b`` in bf16 on cached bf16 copies of the fp32 parameters (what autocast would compute, without
    its per-call casts and dispatch)."""

    @staticmethod
    def forward(ctx, x, w, b):
        ctx.save_for_backward(x, w)
        ctx.has_bias = b is not None
        ctx.b_dtype = b.dtype if b is not None else None
        return _linear_fwd(x, w, b)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        need_db = ctx.has_bias and ctx.needs_input_grad[2]
        dx, dw, db = K.linear_bwd(dy, x, bf16_weight(w), ctx.needs_input_grad[0], ctx.needs_input_grad[1], need_db)
        return (dx if ctx.needs_input_grad[0] else None, dw.to(w.dtype) if ctx.needs_input_grad[1] else None,
                db.to(ctx.b_dtype) if need_db else None)  # fmt: skip


def linear(x, w, b=None):
    if not torch.is_grad_enabled():
        return _linear_fwd(x, w, b)
    return _Linear.apply(x, w, b)


class _LinearPlanes(torch.autograd.Function):
    """``(x w^T)`` stored channel-major ``[n, rows]`` (one plane per output channel)."""

    @staticmethod
    def forward(ctx, x, w):
        x16 = _bf16c(x)
        ctx.save_for_backward(x16, w)
        ctx.x_dtype = x.dtype
        return K.gemm(x16, bf16_weight(w), None, None, None, 0, True)

    @staticmethod
    def backward(ctx, dy):
        x16, w = ctx.saved_tensors
        x2 = x16.reshape(-1, x16.shape[-1])
        d = dy.to(BF16).contiguous()
        dx = mm(d, bf16_weight(w), True, False).view(x16.shape).to(ctx.x_dtype)  # d is [n, rows]: handed over transposed
        return dx, mm(d, x2, False, False, True, 0).to(w.dtype)


def linear_planes(x, w):
    return _LinearPlanes.apply(x, w)


class _SigmoidGateMul(torch.autograd.Function):
    """``sigmoid(x w^T) * other``."""

    @staticmethod
    def forward(ctx, x, w, other):
        x16, o16 = _bf16c(x), _bf16c(other)
        ctx.save_for_backward(x16, w, o16)
        ctx.dtypes = (x.dtype, other.dtype)
        return K.gemm(x16, bf16_weight(w), None, None, o16, 3, False)

    @staticmethod
    def backward(ctx, dy):
        x16, w, o16 = ctx.saved_tensors
        W = bf16_weight(w)
        x2 = x16.reshape(-1, x16.shape[-1])
        n = w.shape[0]
        g = _plain_gemm(x2, W)
        d = dy.reshape(-1, n).to(BF16).contiguous()
        dg, d_other = K.sigmoid_gate_bwd(d, g, o16.reshape(-1, n))  # one pass: dy other s (1 - s) and dy s
        dx = mm(dg, W).view(x16.shape).to(ctx.dtypes[0])
        return dx, _wgrad(dg, x2, w), d_other.view(o16.shape).to(ctx.dtypes[1])


def sigmoid_gate_mul(x, w, other):
    return _SigmoidGateMul.apply(x, w, other)


class _AdaNorm(torch.autograd.Function):
    """``sigmoid(s) * LN(x) + t`` in one kernel each way (LN without affine; ``x`` fp32 or bf16, ``s`` / ``t`` bf16, result
    bf16: the tensor the following projections consume, so no cast kernel runs per projection)."""

    @staticmethod
    def forward(ctx, x, s, t, eps):
        xc, sc = x.contiguous(), s.contiguous()
        y, mean, rstd = K.ada_ln_fwd(xc, sc, t.contiguous(), eps)
        ctx.save_for_backward(xc, sc, mean, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, sc, mean, rstd = ctx.saved_tensors
        d = dy if dy.dtype == BF16 else dy.to(BF16)
        dx, ds = K.ada_ln_bwd(d.contiguous(), xc, sc, mean, rstd)
        return dx, ds, d, None


def ada_norm_supported(x, s, t) -> bool:
    c = x.shape[-1]
    return (x.is_cuda and x.dtype in (torch.float32, BF16) and s.dtype == BF16 and t.dtype == BF16 and s.shape == x.shape
            and t.shape == x.shape and c % 2 == 0 and c <= 1024)


def ada_norm(x, s, t, eps: float = 1e-5):
    return _AdaNorm.apply(x, s, t, eps)


class _GatedResidual(torch.autograd.Function):
    """``a + sigmoid(z) * u``: the gated residual update of the diffusion transformer (``a`` fp32 or bf16, ``z`` / ``u`` bf16)."""

    @staticmethod
    def forward(ctx, a, z, u):
        zc, uc = z.contiguous(), u.contiguous()
        ctx.save_for_backward(zc, uc)
        return K.gated_residual_fwd(a.contiguous(), zc, uc)

    @staticmethod
    def backward(ctx, dy):
        zc, uc = ctx.saved_tensors
        dz, du = K.gated_residual_bwd(dy.contiguous(), zc, uc)
        return dy, dz, du


def gated_residual_supported(a, z, u) -> bool:
    return (a.is_cuda and a.dtype in (torch.float32, BF16) and z.dtype == BF16 and u.dtype == BF16 and z.shape == a.shape
            and u.shape == a.shape and a.numel() % 2 == 0)


def gated_residual(a, z, u):
    return _GatedResidual.apply(a, z, u)


class _Transition(torch.autograd.Function):
    """``swiglu(LN(x) w1^T) w2^T``: LN kernel, GEMM with the SwiGLU epilogue, output GEMM."""

    @staticmethod
    def forward(ctx, x, ln_w, ln_b, w1, w2, eps):
        xc = x.contiguous()
        h, mean, rstd = K.layer_norm_fwd(xc, _f32(ln_w), _f32(ln_b), eps)
        h16 = h if h.dtype == BF16 else h.to(BF16)
        u = K.gemm(h16, bf16_weight(w1), None, None, None, 2, False)
        y = _plain_gemm(u, bf16_weight(w2))
        ctx.save_for_backward(xc, ln_w, ln_b, w1, w2, mean, rstd, h16)
        return y.to(x.dtype) if x.dtype != BF16 else y

    @staticmethod
    def backward(ctx, dy):
        xc, ln_w, ln_b, w1, w2, mean, rstd, h16 = ctx.saved_tensors
        W1, W2 = bf16_weight(w1), bf16_weight(w2)
        c = xc.shape[-1]
        h2 = h16.reshape(-1, c)
        d = dy.reshape(-1, c).to(BF16).contiguous()
        u = K.gemm(h2, W1, None, None, None, 2, False)
        dW2 = _wgrad(d, u, w2)
        dpre = K.gemm(h2, W1, None, None, mm(d, W2), 4, False)  # pre-activations recomputed in the accumulator
        dW1 = _wgrad(dpre, h2, w1)
        dh = mm(dpre, W1).view(xc.shape)
        if xc.dtype != BF16:
            dh = dh.to(xc.dtype)
        need_wb = ln_w is not None and (ctx.needs_input_grad[1] or ctx.needs_input_grad[2])
        dx, partial = K.layer_norm_bwd(dh.contiguous(), xc, _f32(ln_w), mean, rstd, need_wb)
        dlw = dlb = None
        if need_wb:
            sums = partial.sum(0)
            dlw = sums[0].to(ln_w.dtype)
            dlb = sums[1].to(ln_b.dtype) if ln_b is not None else None
        return dx, dlw, dlb, dW1, dW2, None


def transition_supported(x, w1) -> bool:
    return gemm_supported(x, w1) and x.dtype in (BF16, torch.float32) and w1.shape[0] % 2 == 0 and x.shape[-1] <= 1024


def transition(x, ln_w, ln_b, w1, w2, eps: float = 1e-5):
    return _Transition.apply(x, ln_w, ln_b, w1, w2, eps)


class _MatMul(torch.autograd.Function):
    """Differentiable ``op(a) @ op(b)`` on the tcgen05 kernel (2-D or batched 3-D bf16 operands). An operand flagged
    ``trans`` is handed over as stored, ``[.., K, M]`` / ``[.., N, K]``; neither the forward nor the two backward
    products copy or transpose anything: a transposed operand is simply read MN-major by the tensor cores."""

    @staticmethod
    def forward(ctx, a, b, trans_a, trans_b):
        ctx.save_for_backward(a, b)
        ctx.flags = (trans_a, trans_b)
        return mm(a, b, trans_a, trans_b)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        ta, tb = ctx.flags
        d = (dc if dc.dtype == BF16 else dc.to(BF16)).contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = mm(b, d, tb, True) if ta else mm(d, b, False, not tb)
        if ctx.needs_input_grad[1]:
            db = mm(d, a, True, ta) if tb else mm(a, d, not ta, False)
        return da, db, None, None


def matmul(a, b, trans_a: bool = False, trans_b: bool = False):
    """Differentiable product on the own GEMM kernel; see ``_MatMul``."""
    return _MatMul.apply(a, b, bool(trans_a), bool(trans_b))


def msa_weighted_average(w, v):
    """``out[b,s,q,h,:] = sum_k w[b,h,q,k] v[b,s,k,h,:]``: one [N, N] x [N, S * d] product per (batch, head), the pair
    weights shared by all MSA rows (reference: model/attention.py:272-341)."""
    B, S, N, H, D = v.shape
    vp = v.permute(0, 3, 2, 1, 4).reshape(B * H, N, S * D)  # keys as rows, (row, channel) as columns
    out = matmul(w.reshape(B * H, N, N).to(BF16), vp.to(BF16))
    return out.view(B, H, N, S, D).permute(0, 3, 2, 1, 4)


def outer_product_mean(a, b, out_w, out_b, mask, eps: float = 1e-3, row_chunk: int = 96, mask_i=None, mask_j=None):
    """``(sum_s a[s,i,:] (x) b[s,j,:]) . out_w + out_b`` over valid rows, as two tensor-core products per block of
    ``row_chunk`` tokens i: first the [chunk * E, S] x [S, N * E] contraction over the MSA rows, then, after bringing the
    two feature axes together, the [chunk * N, E * E] x [E * E, C] projection. The full ``[N, N, E, E]`` outer product
    never exists at once (reference: model/ops.py:683-785, tiled form model/tiled_linear.py:67-88). ``a`` and ``b`` may
    cover different token ranges (a block of the output); their row masks are then ``mask_i`` / ``mask_j``."""
    B, S, Ni, E = a.shape
    Nj = b.shape[2]
    C = out_w.shape[-1]
    w2 = out_w.reshape(E * E, C).to(BF16)  # a differentiable cast: the projection weight trains through it
    a16, b16 = a.to(BF16), b.to(BF16)
    mi16 = (mask if mask_i is None else mask_i).to(BF16)
    mj16 = (mask if mask_j is None else mask_j).to(BF16)
    outs = []
    for bi in range(B):
        bm = b16[bi].reshape(S, Nj * E)
        count = mm(mi16[bi], mj16[bi], True, False, True)  # [Ni, Nj] valid rows per pair, exact in fp32
        rows = []
        for i0 in range(0, Ni, row_chunk):
            i1 = min(Ni, i0 + row_chunk)
            am = a16[bi, :, i0:i1].reshape(S, (i1 - i0) * E)
            ab = matmul(am, bm, True, False)  # [(i, e), (j, f)]
            ab = ab.view(i1 - i0, E, Nj, E).permute(0, 2, 1, 3).reshape((i1 - i0) * Nj, E * E)
            rows.append(matmul(ab, w2).view(i1 - i0, Nj, C))
        act = torch.cat(rows, 0) + out_b.to(BF16)
        outs.append(act / (eps + count).unsqueeze(-1).to(act.dtype))
    return torch.stack(outs, 0)


class _PlaneContract(torch.autograd.Function):
    """Triangle contraction on channel-major planes ``[2, P, N, N]`` (a = planes[0], b = planes[1], P = channels x
    batch): outgoing ``act[p] = a[p] b[p]^T``, incoming ``act[p] = b[p]^T a[p]``. Forward and both operand gradients
    are batched tcgen05 products that read the planes as they lie (transposed operands are MN-major MMA operands);
    the two gradients are written straight into the halves of one ``[2, P, N, N]`` tensor."""

    @staticmethod
    def forward(ctx, planes, outgoing):
        a, b = planes[0], planes[1]
        ctx.save_for_backward(planes)
        ctx.outgoing = outgoing
        return mm(a, b, False, True) if outgoing else mm(b, a, True, False)

    @staticmethod
    def backward(ctx, d_act):
        (planes,) = ctx.saved_tensors
        a, b = planes[0], planes[1]
        d = d_act if d_act.dtype == BF16 else d_act.to(BF16)
        d = d.contiguous()
        grads = torch.empty_like(planes)
        if ctx.outgoing:  # act = a b^T: da = d b, db = d^T a
            mm(d, b, False, False, out=grads[0])
            mm(d, a, True, False, out=grads[1])
        else:  # act = b^T a: da = b d, db = a d^T
            mm(b, d, False, False, out=grads[0])
            mm(a, d, False, True, out=grads[1])
        return grads, None


def plane_contract(planes, outgoing: bool):
    return _PlaneContract.apply(planes, bool(outgoing))


# ------------------------------------------------------------------------------------------------
# Pair-bias attention: tcgen05 forward kernel and one fused tcgen05 backward kernel (dQ, dK, dV accumulated in tensor
# memory, logits recomputed in fp32). Shapes beyond the tensor-memory budget of the fused backward (long rows) fall back
# to row chunks sized for L2; a negative DF3_ATTN_BWD_CHUNK_MB forces that chunked form everywhere (for comparisons).
ATTN_BWD_CHUNK_BYTES = int(os.environ.get("DF3_ATTN_BWD_CHUNK_MB", "40")) * 1024 * 1024


def attention_supported(q, k, v, bias) -> bool:
    d = q.shape[-1]
    # the chunked backward (rows beyond the fused kernel's tensor-memory budget) handles keys in pairs
    even = q.shape[-2] % 2 == 0 or not torch.is_grad_enabled() or K.attention_bwd_fused_supported(q.shape[-2], d)
    return (q.is_cuda and q.dim() == 5 and q.shape == k.shape and q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16
            and d % 8 == 0 and d <= 64 and even)


def window_attention_supported(q, k, v, bias) -> bool:
    """Atom-window attention on the pair-bias attention kernel: ``q`` ``[B, S, W, H, Q, D]``, ``k``/``v``
    ``[B, S, W, H, K, D]`` in bf16, ``bias`` ``[B, 1, W, H, Q, K]`` (shared by the S samples, key mask folded in).
    Forward only: with gradients wanted the PyTorch statement runs under autograd."""
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v, bias)):
        return False
    if not (q.is_cuda and q.dim() == 6 and k.dim() == 6 and bias.dim() == 6 and k.shape == v.shape):
        return False
    if not (q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16 and bias.dtype in (BF16, torch.float32)):
        return False
    B, S, W, H, Q, D = q.shape
    keys = k.shape[-2]
    return (k.shape[:4] == q.shape[:4] and k.shape[-1] == D and D % 8 == 0 and D <= 64 and keys % 8 == 0
            and tuple(bias.shape) == (B, 1, W, H, Q, keys))


@torch.no_grad()
def window_attention(q, k, v, bias, scale: float):
    """One launch per batch element: windows become the kernel's batch axis and samples its row axis, so the bias tile of
    a window (staged by TMA when bf16) serves all samples (reference: atom_cross_attn.py:764-769, there three library
    calls over a materialised ``[.., H, Q, K]`` fp32 logit tensor). The 32 queries of a window fill a quarter of the
    kernel's 128-row tile; the work is bound by launch count and memory traffic, not by the tensor pipe."""
    outs = []
    for b in range(q.shape[0]):
        out, _ = K.attention_fwd(q[b].transpose(0, 1), k[b].transpose(0, 1), v[b].transpose(0, 1), bias[b, 0], None, scale, False)
        outs.append(out.transpose(0, 1))  # [S, W, H, Q, D] in q's memory order
    return outs[0].unsqueeze(0) if len(outs) == 1 else torch.stack(outs)


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, bias, key_mask, scale):
        if any(ctx.needs_input_grad[:4]):
            out, lse, out32 = K.attention_fwd_train(q, k, v, bias, key_mask, scale)  # out32: unrounded O for the row sums
        else:
            out, lse = K.attention_fwd(q, k, v, bias, key_mask, scale, False)
            out32 = out
        ctx.save_for_backward(q, k, v, bias, key_mask, out32, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, d_out):
        q, k, v, bias, key_mask, out, lse = ctx.saved_tensors
        want_bias = bias is not None and ctx.needs_input_grad[3]
        dq, dk, dv, dbias = K.attention_bwd(q, k, v, out, d_out, bias, key_mask, lse, ctx.scale, want_bias,
                                            ATTN_BWD_CHUNK_BYTES)  # fmt: skip
        return dq, dk, dv, (dbias.to(bias.dtype) if want_bias else None), None, None


def pair_bias_attention(q, k, v, bias, key_mask, scale: float):
    return _Attention.apply(q, k, v, bias, key_mask, float(scale))


def window_attention_train_supported(q, k, v, bias) -> bool:
    """Atom-window attention with gradients: the queries of a window are padded up to its key count and the call runs
    on the training forward and the fused backward of the pair-bias attention (padded rows receive no gradient and
    give none). Needs bf16 operands, more keys than queries, and a key count the fused backward holds in tensor memory."""
    if not (q.is_cuda and q.dim() == 6 and k.dim() == 6 and bias.dim() == 6 and k.shape == v.shape):
        return False
    if not (q.dtype == BF16 and k.dtype == BF16 and v.dtype == BF16 and bias.dtype in (BF16, torch.float32)):
        return False
    B, S, W, H, Q, D = q.shape
    keys = k.shape[-2]
    return (k.shape[:4] == q.shape[:4] and k.shape[-1] == D and D % 8 == 0 and D <= 64 and keys % 8 == 0 and Q <= keys
            and tuple(bias.shape) == (B, 1, W, H, Q, keys) and bool(K.attention_bwd_fused_supported(keys, D)))


def window_attention_train(q, k, v, bias, scale: float):
    """``q`` ``[B, S, W, H, Q, D]`` (a head-major view of the projection ``[B, S, W, Q, H, D]``), ``k`` / ``v``
    ``[B, S, W, H, K, D]``, ``bias`` ``[B, 1, W, H, Q, K]``. Windows become the batch axis and samples the row axis of the
    attention op, so the bias gradient is summed over the samples inside the backward kernel."""
    B, S, W, H, Q, D = q.shape
    keys = k.shape[-2]
    outs = []
    for b in range(B):
        qb = q[b].permute(0, 1, 3, 2, 4)  # [S, W, Q, H, D]: the projection's own memory order when q is the usual view
        qp = torch.nn.functional.pad(qb, (0, 0, 0, 0, 0, keys - Q)).permute(1, 0, 3, 2, 4)  # [W, S, H, keys, D]
        bp = torch.nn.functional.pad(bias[b, 0], (0, 0, 0, keys - Q))  # [W, H, keys, keys]
        out = pair_bias_attention(qp, k[b].transpose(0, 1), v[b].transpose(0, 1), bp, None, scale)  # [W, S, H, keys, D]
        outs.append(out[..., :Q, :].transpose(0, 1))
    return outs[0].unsqueeze(0) if len(outs) == 1 else torch.stack(outs)


def _grid_heads(t, transpose: bool):
    """[B, N1, N2, H, D] -> [B, R, H, L, D] (a view): R is the axis attention does not mix."""
    return t.permute(0, 2, 3, 1, 4) if transpose else t.permute(0, 1, 3, 2, 4)


class _GridAttentionPacked(torch.autograd.Function):
    """Row / column attention on the packed projection ``qkv`` [B, N, N, 3, H, D].

    Taking the packed tensor keeps the split out of autograd: backward writes dq, dk and dv straight into the three
    slots of one gradient tensor (three strided copies) instead of three zero-filled full-size tensors that are then
    added together.
    """

    @staticmethod
    def forward(ctx, qkv, bias, key_mask, scale, transpose):
        q, k, v = (_grid_heads(qkv[:, :, :, i], transpose) for i in range(3))
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            out, lse, out32 = K.attention_fwd_train(q, k, v, bias, key_mask, scale)
        else:
            out, lse = K.attention_fwd(q, k, v, bias, key_mask, scale, False)
            out32 = out
        ctx.save_for_backward(qkv, bias, key_mask, out32, lse)
        ctx.scale, ctx.transpose = scale, transpose
        return out

    @staticmethod
    def backward(ctx, d_out):
        qkv, bias, key_mask, out, lse = ctx.saved_tensors
        q, k, v = (_grid_heads(qkv[:, :, :, i], ctx.transpose) for i in range(3))
        want_bias = bias is not None and ctx.needs_input_grad[1]
        dqkv = torch.empty_like(qkv)
        if ATTN_BWD_CHUNK_BYTES >= 0 and K.attention_bwd_fused_supported(q.shape[3], q.shape[4]):
            # the fused kernel writes the three gradients straight into their slots of the packed tensor
            dq, dk, dv = (_grid_heads(dqkv[:, :, :, i], ctx.transpose) for i in range(3))
            dbias = K.attention_bwd_into(q, k, v, out, d_out, bias, key_mask, lse, ctx.scale, want_bias, dq, dk, dv)
        else:
            dq, dk, dv, dbias = K.attention_bwd(q, k, v, out, d_out, bias, key_mask, lse, ctx.scale, want_bias,
                                                ATTN_BWD_CHUNK_BYTES)  # fmt: skip
            for i, g in enumerate((dq, dk, dv)):
                _grid_heads(dqkv[:, :, :, i], ctx.transpose).copy_(g)
        return dqkv, (dbias.to(bias.dtype) if want_bias else None), None, None, None


def grid_attention_packed(qkv, bias, key_mask, scale: float, transpose: bool):
    return _GridAttentionPacked.apply(qkv, bias, key_mask, float(scale), bool(transpose))


def check_status() -> None:
    """Raise if a kernel's bounded wait ran out since the last check (synchronises the device)."""
    code = K.gemm_status() or K.elementwise_status()
    if code != 0:
        raise RuntimeError(f"deepfold3_dev_b200: a kernel wait timed out (status {code}); results of this step are invalid")
