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
    if nat is not None and nat.has("transition") and nat.transition_supported(x, w1):
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


def window_attention(q, k, v, bias, scale: float):
    nat = _native(q)
    if nat is not None and nat.has("window_attention") and nat.window_attention_supported(q, k, v, bias):
        _CENSUS["window_attention:sm100"] += 1
        return nat.window_attention(q, k, v, bias, scale)
    _CENSUS["window_attention:torch"] += 1
    return ref.window_attention(q, k, v, bias, scale)


def triangle_contract(a, b, outgoing: bool):
    nat = _native(a)
    if nat is not None and nat.has("triangle_contract") and nat.contract_supported(a):
        _CENSUS["triangle_contract:sm100"] += 1
        return nat.triangle_contract(a, b, outgoing)
    _CENSUS["triangle_contract:torch"] += 1
    return ref.triangle_contract(a, b, outgoing)


def gated_dual_linear(x, w_gate, w_proj, mask=None):
    nat = _native(x)
    if nat is not None and nat.has("gated_dual_linear") and nat.gemm_supported(x, w_gate):
        _CENSUS["gated_dual_linear:sm100"] += 1
        return nat.gated_dual_linear(x, w_gate, w_proj, mask)
    _CENSUS["gated_dual_linear:torch"] += 1
    return ref.gated_dual_linear(x, w_gate, w_proj, mask)


def linear(x, w, b=None):
    nat = _native(x)
    if nat is not None and nat.has("linear") and nat.gemm_supported(x, w):
        _CENSUS["linear:sm100"] += 1
        return nat.linear(x, w, b)
    _CENSUS["linear:torch"] += 1
    return torch.nn.functional.linear(x, w, b)


def outer_product_mean(a, b, out_w, out_b, mask, eps: float = 1e-3, mask_i=None, mask_j=None):
    _CENSUS["outer_product_mean:torch"] += 1
    return ref.outer_product_mean(a, b, out_w, out_b, mask, eps, mask_i, mask_j)


def msa_weighted_average(w, v):
    _CENSUS["msa_weighted_average:torch"] += 1
    return ref.msa_weighted_average(w, v)
