"""Fused operators of the model.

Every function here has two bodies that compute the same thing: the sm_100a
CUDA kernel (``ops/csrc`` through ``ops/native.py``) for CUDA tensors, and the
PyTorch statement in ``ops/reference.py`` for CPU tensors and as the test
oracle. On a machine with a GPU the extension must load: a missing extension
raises instead of silently computing on the fallback.

``census()`` reports how often each op took which body, the equivalent of the
reference's per-site kernel census (model/kernel_census.py:45-135).
"""

from __future__ import annotations

import collections

import os

import torch

from . import reference as ref

_CENSUS: collections.Counter = collections.Counter()


def census(reset: bool = False) -> dict[str, int]:
    out = dict(_CENSUS)
    if reset:
        _CENSUS.clear()
    return out


def _native(x: torch.Tensor):
    """The native module when ``x`` lives on a GPU, else ``None``."""
    if not x.is_cuda:
        return None
    from . import native

    return native.require()


def _autocast_dtype(x: torch.Tensor):
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type)
    return None


def bf16_mode(x: torch.Tensor) -> bool:
    """True when ``x`` is a CUDA tensor that is bf16 or sits under bf16 autocast: the tensor-core kernels apply."""
    return x.is_cuda and (x.dtype == torch.bfloat16 or _autocast_dtype(x) == torch.bfloat16)


def fused(x: torch.Tensor, feature: str):
    """The native namespace if ``feature`` may run on ``x``, else ``None``."""
    if not x.is_cuda or not bf16_mode(x):
        return None
    nat = _native(x)
    return nat if nat.has(feature) else None


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    nat = _native(x)
    if nat is not None and nat.has("layer_norm") and x.dtype in (torch.bfloat16, torch.float32):
        _CENSUS["layer_norm:sm100"] += 1
        return nat.layer_norm(x, weight, bias, eps)
    _CENSUS["layer_norm:torch"] += 1
    return ref.layer_norm(x, weight, bias, eps)


def swiglu(x):
    nat = _native(x)
    if nat is not None and nat.has("swiglu") and x.dtype in (torch.bfloat16, torch.float32):
        _CENSUS["swiglu:sm100"] += 1
        return nat.swiglu(x)
    _CENSUS["swiglu:torch"] += 1
    return ref.swiglu(x)


def transition(x, ln_w, ln_b, w1, w2, eps: float = 1e-5):
    nat = _native(x)
    if nat is not None and bf16_mode(x) and nat.has("transition") and nat.transition_supported(x, w1):
        _CENSUS["transition:sm100"] += 1
        return nat.transition(x, ln_w, ln_b, w1, w2, eps)
    _CENSUS["transition:torch"] += 1
    h = torch.nn.functional.linear(layer_norm(x, ln_w, ln_b, eps), w1)
    return torch.nn.functional.linear(swiglu(h), w2)


def dropout_add(residual, x, p: float, training: bool, share_dim: int):
    if not training or p == 0.0:
        return residual + x
    nat = _native(x)
    if nat is not None and nat.has("dropout_add") and x.dtype == residual.dtype:
        _CENSUS["dropout_add:sm100"] += 1
        return nat.dropout_add(residual, x, p, share_dim)
    _CENSUS["dropout_add:torch"] += 1
    return ref.dropout_add(residual, x, p, training, share_dim)


def pair_bias_attention(q, k, v, bias, key_mask, scale: float, fp32_qk: bool = False):
    nat = _native(q)
    if nat is not None and nat.has("pair_bias_attention") and nat.attention_supported(q, k, v, bias):
        _CENSUS["pair_bias_attention:sm100"] += 1
        return nat.pair_bias_attention(q, k, v, bias, key_mask, scale)
    _CENSUS["pair_bias_attention:torch"] += 1
    return ref.pair_bias_attention(q, k, v, bias, key_mask, scale, fp32_qk)


def grid_attention(qkv, bias, key_mask, scale: float, transpose: bool):
    """Row (``transpose=False``) or column attention of the pair tensor from the packed projection [B, N, N, 3, H, D].

    Returns [B, R, H, L, D] like ``pair_bias_attention`` on the three permuted slices, which is also the fallback.
    """
    nat = _native(qkv)
    heads = (lambda t: t.permute(0, 2, 3, 1, 4)) if transpose else (lambda t: t.permute(0, 1, 3, 2, 4))
    q, k, v = (heads(qkv[:, :, :, i]) for i in range(3))
    if (nat is not None and nat.has("pair_bias_attention") and "grid_attention_packed" not in os.environ.get("DF3_DISABLE_OPS", "") and qkv.is_contiguous()
            and torch.is_grad_enabled() and qkv.requires_grad and nat.attention_supported(q, k, v, bias)):
        _CENSUS["pair_bias_attention:sm100"] += 1
        return nat.grid_attention_packed(qkv, bias, key_mask, scale, transpose)
    return pair_bias_attention(q, k, v, bias, key_mask, scale)


def window_attention(q, k, v, bias, scale: float):
    nat = _native(q)
    if nat is not None and nat.has("window_attention") and nat.window_attention_supported(q, k, v, bias):
        _CENSUS["window_attention:sm100"] += 1
        return nat.window_attention(q, k, v, bias, scale)
    # With gradients the kernels are opt-in (DF3_WINDOW_ATTENTION_TRAIN=1): padding the 32 queries of a window to its 128
    # keys makes the training forward and the fused backward do four times the row work, and at crop 384 with 48 samples
    # the step came out 6 ms slower than with the PyTorch statement (814.8 against 820.6 ms on one B200). What the
    # kernels save is memory: no fp32 logit tensor per block is kept for the backward.
    if (nat is not None and nat.has("window_attention") and torch.is_grad_enabled() and os.environ.get("DF3_WINDOW_ATTENTION_TRAIN", "0") == "1"
            and nat.window_attention_train_supported(q, k, v, bias)):
        _CENSUS["window_attention_train:sm100"] += 1
        return nat.window_attention_train(q, k, v, bias, scale)
    _CENSUS["window_attention:torch"] += 1
    return ref.window_attention(q, k, v, bias, scale)


def _plane_contract(nat, planes, outgoing: bool):
    """One N x N x N product per channel plane (reference: model/triton/fused_trimul.py:264-279, there a library
    batched GEMM); on the tcgen05 kernel when the token count keeps plane rows 16-byte aligned."""
    if nat.has("matmul") and planes.shape[-1] % 8 == 0:
        _CENSUS["triangle_plane_contract:sm100"] += 1
        return nat.plane_contract(planes, outgoing)
    _CENSUS["triangle_plane_contract:torch"] += 1
    a, b = planes[0], planes[1]
    return torch.bmm(a, b.transpose(1, 2)) if outgoing else torch.bmm(b.transpose(1, 2), a)


def triangle_contract_norm(z0, w_gate, w_proj, mask, outgoing: bool, ln_w, ln_b, eps: float = 1e-5):
    """``LN_c(triangle_projection_contract(...))``: on the GPU the contraction result stays channel-major and one kernel
    normalises and transposes it to channel-last."""
    nat = fused(z0, "gated_dual_linear")
    C = w_gate.shape[0] // 2
    if nat is not None and nat.has("plane_layer_norm") and nat.gemm_supported(z0, w_gate) and C in (32, 64, 128, 256):
        _CENSUS["triangle_contract_norm:sm100"] += 1
        B, N = z0.shape[0], z0.shape[1]
        planes = nat.gated_dual_linear(z0, w_gate, w_proj, mask, True, True).view(2, C * B, N, N)
        act = _plane_contract(nat, planes, outgoing)
        return nat.plane_layer_norm(act.view(C, B * N * N), ln_w, ln_b, eps).view(B, N, N, C)
    return layer_norm(triangle_projection_contract(z0, w_gate, w_proj, mask, outgoing), ln_w, ln_b, eps)


def triangle_projection_contract(z0, w_gate, w_proj, mask, outgoing: bool):
    """Gated a/b projection of the triangle multiply followed by the contraction over the third token.

    ``w_gate``/``w_proj`` hold the a channels on even rows and the b channels on odd rows
    (reference: ops.py:318-392). Returns ``[B, N, N, C]``.
    """
    nat = fused(z0, "gated_dual_linear")
    if nat is not None and nat.gemm_supported(z0, w_gate):
        _CENSUS["triangle_projection_contract:sm100"] += 1
        B, N = z0.shape[0], z0.shape[1]
        C = w_gate.shape[0] // 2
        planes = nat.gated_dual_linear(z0, w_gate, w_proj, mask, True, True).view(2, C * B, N, N)
        act = _plane_contract(nat, planes, outgoing)
        return act.view(C, B, N, N).permute(1, 2, 3, 0)
    ab = gated_dual_linear(z0, w_gate, w_proj, mask)
    return triangle_contract(ab[..., 0::2], ab[..., 1::2], outgoing)


def triangle_contract(a, b, outgoing: bool):
    nat = _native(a)
    if nat is not None and nat.has("triangle_contract") and nat.contract_supported(a):
        _CENSUS["triangle_contract:sm100"] += 1
        return nat.triangle_contract(a, b, outgoing)
    _CENSUS["triangle_contract:torch"] += 1
    return ref.triangle_contract(a, b, outgoing)


def gated_dual_linear(x, w_gate, w_proj, mask=None):
    nat = _native(x)
    if nat is not None and bf16_mode(x) and nat.has("gated_dual_linear") and nat.gemm_supported(x, w_gate):
        _CENSUS["gated_dual_linear:sm100"] += 1
        return nat.gated_dual_linear(x, w_gate, w_proj, mask)
    _CENSUS["gated_dual_linear:torch"] += 1
    return ref.gated_dual_linear(x, w_gate, w_proj, mask)


def sigmoid_gate_mul(x, w, other):
    """``sigmoid(x w^T) * other`` (the output gates of the triangle and attention blocks)."""
    nat = fused(x, "sigmoid_gate_mul")
    if nat is not None and nat.gemm_supported(x, w) and other.shape[-1] == w.shape[0]:
        _CENSUS["sigmoid_gate_mul:sm100"] += 1
        return nat.sigmoid_gate_mul(x, w, other)
    _CENSUS["sigmoid_gate_mul:torch"] += 1
    return torch.sigmoid(torch.nn.functional.linear(x, w)) * other


def ada_norm(x, s_pre, t, eps: float = 1e-5):
    """Adaptive LayerNorm ``sigmoid(s_pre) * LN(x) + t`` (LN without affine parameters; AF3 algorithm 26, the form
    inside every diffusion transformer block). One kernel each way when the conditioning tensors are bf16 and shaped
    like ``x``; the result is then bf16."""
    nat = fused(x, "ada_norm")
    if nat is not None and nat.ada_norm_supported(x, s_pre, t):
        _CENSUS["ada_norm:sm100"] += 1
        return nat.ada_norm(x, s_pre, t, eps)
    _CENSUS["ada_norm:torch"] += 1
    return torch.sigmoid(s_pre) * layer_norm(x, None, None, eps) + t


def gated_residual(a, z, u):
    """``a + sigmoid(z) * u``: a residual update behind a sigmoid gate."""
    nat = fused(a, "ada_norm")
    if nat is not None and nat.gated_residual_supported(a, z, u):
        _CENSUS["gated_residual:sm100"] += 1
        return nat.gated_residual(a, z, u)
    _CENSUS["gated_residual:torch"] += 1
    return a + torch.sigmoid(z) * u


def head_bias_planes(x, w):
    """Per-head additive attention bias ``[B, H, R, N]`` from the pair rows ``x [B, R, N, C]``, ``w [H, C]``."""
    nat = fused(x, "linear_planes")
    if nat is not None and nat.gemm_supported(x, w):
        _CENSUS["head_bias_planes:sm100"] += 1
        B, R, N = x.shape[0], x.shape[1], x.shape[2]
        return nat.linear_planes(x, w).view(w.shape[0], B, R, N).transpose(0, 1)
    _CENSUS["head_bias_planes:torch"] += 1
    return torch.nn.functional.linear(x, w).permute(0, 3, 1, 2)


def stacked_linear(x, *ws):
    """``[x w_0^T, x w_1^T, ...]`` concatenated on the last axis, as one GEMM."""
    nat = fused(x, "gemm")
    if nat is not None:
        _CENSUS["stacked_linear:sm100"] += 1
        return nat.stacked_linear(x, *ws)
    _CENSUS["stacked_linear:torch"] += 1
    return torch.cat([torch.nn.functional.linear(x, w) for w in ws], -1)


def linear(x, w, b=None):
    """``x w^T + b``; in bf16 mode on cached bf16 copies of the parameters, else ``F.linear``."""
    if x.is_cuda and w.dtype == torch.float32 and x.dim() >= 2 and x.numel() > 0:
        nat = fused(x, "gemm")
        if nat is not None:
            _CENSUS["linear:bf16_cached"] += 1
            return nat.linear(x, w, b)
    _CENSUS["linear:torch"] += 1
    return torch.nn.functional.linear(x, w, b)


def outer_product_mean(a, b, out_w, out_b, mask, eps: float = 1e-3, mask_i=None, mask_j=None):
    """MSA outer-product mean. bf16 CUDA inputs with 8-aligned extents run as tensor-core products on the own GEMM
    kernel (contraction over MSA rows, then the projection), blocked over tokens; everything else takes the fp32
    statement."""
    nat = fused(a, "matmul")
    have_masks = mask is not None or (mask_i is not None and mask_j is not None)
    if (nat is not None and have_masks and a.shape[1] % 8 == 0 and (a.shape[2] * a.shape[3]) % 8 == 0 and a.shape[2] % 8 == 0
            and b.shape[2] % 8 == 0 and out_w.shape[-1] % 8 == 0):
        _CENSUS["outer_product_mean:sm100"] += 1
        return nat.outer_product_mean(a, b, out_w, out_b, mask, eps, mask_i=mask_i, mask_j=mask_j)
    _CENSUS["outer_product_mean:torch"] += 1
    return ref.outer_product_mean(a, b, out_w, out_b, mask, eps, mask_i, mask_j)


def msa_weighted_average(w, v):
    """Pair-weighted average over keys for every MSA row: on the GPU one batched tensor-core product per head."""
    nat = fused(v, "matmul")
    if nat is not None and v.shape[2] % 8 == 0 and (v.shape[1] * v.shape[4]) % 8 == 0:
        _CENSUS["msa_weighted_average:sm100"] += 1
        return nat.msa_weighted_average(w, v)
    _CENSUS["msa_weighted_average:torch"] += 1
    return ref.msa_weighted_average(w, v)
