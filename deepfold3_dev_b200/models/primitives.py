"""Building blocks shared by every model family: linears, norms, transitions.

Parameter names and shapes equal the reference's (model/primitives.py:47-306)
so state dicts interchange. The arithmetic of each block is delegated to
``deepfold3_dev_b200.ops`` so that CUDA tensors run the sm_100a kernels and
CPU tensors run the fp32 PyTorch statement of the same math.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops

# std of a unit normal truncated at +-2 sigma; divides the target std so the
# truncated draw has the wanted variance (AF3 initialisers).
TRUNCATED_NORMAL_STDDEV_FACTOR = 0.87962566103423978


def block_residual_scale(layer_idx: int, num_layer: int, per_layer: bool, uniform: bool) -> float:
    """Multiplier on each branch output of block ``layer_idx`` (reference: primitives.py:20-44)."""
    if per_layer and uniform:
        raise ValueError("residual_output_scaling and uniform_residual_scale are mutually exclusive on the same stack")
    if per_layer:
        return 1.0 / math.sqrt(layer_idx + 1.0)
    if uniform:
        return 1.0 / math.sqrt(float(num_layer))
    return 1.0


class Gain:
    """A branch multiplier that costs nothing when it is 1: ``Gain(s) * x`` is ``x`` itself for ``s == 1``."""

    __slots__ = ("value",)

    def __init__(self, value: float):
        self.value = float(value)

    def __mul__(self, x):
        return x if self.value == 1.0 else x * self.value


def af3_linear_init_(weight: torch.Tensor, initializer: str = "linear") -> None:
    """AF3 variance-scaling init: ``zeros``, or truncated normal with var 1/fan_in (``relu``: 2/fan_in)."""
    if initializer == "zeros":
        nn.init.zeros_(weight)
        return
    fan_in = weight.shape[1] if weight.dim() >= 2 else weight.shape[0]
    var = (2.0 if initializer == "relu" else 1.0) / fan_in
    nn.init.trunc_normal_(weight, mean=0.0, std=math.sqrt(var) / TRUNCATED_NORMAL_STDDEV_FACTOR, a=-2.0, b=2.0)


def small_normal_init_(weight: torch.Tensor, target: float) -> None:
    """Truncated normal whose output std is about ``target`` for unit-variance input."""
    std = float(target) / math.sqrt(weight.shape[1]) / TRUNCATED_NORMAL_STDDEV_FACTOR
    nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-2.0, b=2.0)


class Linear(nn.Linear):
    """``nn.Linear`` whose product goes through ``ops.linear`` (bf16 on cached weight copies on the GPU)."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, self.bias)


class LinearNoBias(Linear):
    """Bias-free linear with AF3 initialisation."""

    def __init__(self, in_features: int, out_features: int, initializer: str = "linear"):
        super().__init__(in_features, out_features, bias=False)
        af3_linear_init_(self.weight, initializer)


def biased_linear(in_features: int, out_features: int, initializer: str = "linear", bias_value: float = 0.0):
    lin = Linear(in_features, out_features)
    af3_linear_init_(lin.weight, initializer)
    nn.init.constant_(lin.bias, bias_value)
    return lin


def layer_norm(x, normalized_shape=None, weight=None, bias=None, eps: float = 1e-5):
    """LayerNorm over the last axis with fp32 statistics, result in ``x.dtype``."""
    return ops.layer_norm(x, weight, bias, eps)


def rms_normalize(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return F.rms_norm(x, (x.shape[-1],), eps=eps)


class LayerNorm(nn.LayerNorm):
    """``nn.LayerNorm`` whose forward keeps the statistics in fp32 under autocast."""

    def __init__(self, normalized_shape, *, eps=1e-5, elementwise_affine=True, bias=True, output_scale: float = 1.0):
        super().__init__(normalized_shape, eps=eps, elementwise_affine=elementwise_affine, bias=bias)
        self.output_scale = float(output_scale)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = ops.layer_norm(x, self.weight, self.bias, self.eps)
        return y if self.output_scale == 1.0 else y * self.output_scale


class AdaLayerNorm(nn.Module):
    """LN(x) scaled and shifted by projections of a conditioning vector (reference: primitives.py:158-190)."""

    def __init__(self, dim: int, cond_dim: int):
        super().__init__()
        self.norm = LayerNorm(dim, elementwise_affine=False)
        self.cond_norm = LayerNorm(cond_dim, elementwise_affine=False, bias=False)
        self.cond_norm_weight = nn.Parameter(torch.ones(cond_dim))
        self.cond_scale = biased_linear(cond_dim, dim, "zeros")
        self.cond_bias = LinearNoBias(cond_dim, dim, initializer="zeros")

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        c = ops.layer_norm(cond, self.cond_norm_weight, None)
        return torch.sigmoid(self.cond_scale(c)) * self.norm(x) + self.cond_bias(c)


class SwiGLU(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.swiglu(x)


class TransitionBlock(nn.Module):
    """``W2 · swiglu(W1 · LN(x))`` (reference: primitives.py:201-251).

    ``linear1`` maps c → 2·f·c, ``linear2`` maps f·c → c and starts at zero
    unless ``linear_out_init_gain`` asks for a scaled orthogonal start.
    """

    def __init__(self, channels, num_intermediate_factor=4, optim=None, linear_out_init_gain=None):
        super().__init__()
        hidden = channels * num_intermediate_factor
        self.norm = LayerNorm(channels)
        self.linear1 = LinearNoBias(channels, hidden * 2, initializer="relu")
        self.linear2 = LinearNoBias(hidden, channels, initializer="zeros")
        if linear_out_init_gain is not None:
            nn.init.orthogonal_(self.linear2.weight, gain=float(linear_out_init_gain))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.transition(x, self.norm.weight, self.norm.bias, self.linear1.weight, self.linear2.weight, self.norm.eps)


class AdaTransitionBlock(nn.Module):
    """AdaLN-zero feed-forward of the diffusion stacks (reference: primitives.py:254-306)."""

    def __init__(self, channels, cond_dim, num_intermediate_factor=2, optim=None):
        super().__init__()
        hidden = channels * num_intermediate_factor
        self.norm = LayerNorm(channels, elementwise_affine=False)
        self.cond_norm_weight = nn.Parameter(torch.ones(cond_dim))
        self.cond_scale = biased_linear(cond_dim, channels, "zeros")
        self.cond_bias = LinearNoBias(cond_dim, channels, initializer="zeros")
        self.linear1 = LinearNoBias(channels, hidden * 2, initializer="relu")
        self.linear2 = LinearNoBias(hidden, channels, initializer="zeros")
        self.zero_cond = biased_linear(cond_dim, channels, "zeros", bias_value=-2.0)

    def forward(self, x: torch.Tensor, cond: torch.Tensor) -> torch.Tensor:
        c = ops.layer_norm(cond, self.cond_norm_weight, None)
        xn = torch.sigmoid(self.cond_scale(c)) * ops.layer_norm(x) + self.cond_bias(c)
        out = self.linear2(ops.swiglu(self.linear1(xn)))
        return torch.sigmoid(self.zero_cond(cond)) * out


def make_transition_block(channels, num_intermediate_factor=4, config=None, linear_out_init_gain=None):
    """Factory kept for API parity (reference: model/optim.py:50-105); one implementation here."""
    return TransitionBlock(channels, num_intermediate_factor, linear_out_init_gain=linear_out_init_gain)


def make_ada_transition_block(channels, cond_dim, num_intermediate_factor=2, config=None):
    return AdaTransitionBlock(channels, cond_dim, num_intermediate_factor)


# --- row chunking for inference under a byte budget (reference: primitives.py:309-388) ---


def gemm_itemsize(x: torch.Tensor) -> int:
    if torch.is_autocast_enabled(x.device.type):
        return torch.get_autocast_dtype(x.device.type).itemsize
    return x.element_size()


def budget_rows(budget: int, n: int, bytes_per_position: int) -> int:
    """Rows per chunk so a ``[rows, n]`` slab of ``bytes_per_position`` stays within ``budget``; 0 = no chunking."""
    if budget <= 0:
        return 0
    rows = budget // (n * bytes_per_position)
    if rows >= n:
        return 0
    return 1 << (max(rows, 1).bit_length() - 1)


def map_row_chunks(fn, x: torch.Tensor, chunk: int, *more: torch.Tensor) -> torch.Tensor:
    """``fn(x, *more)`` evaluated ``chunk`` rows of dim -3 at a time (inference only)."""
    rows = x.shape[-3]
    if chunk <= 0 or rows <= chunk or torch.is_grad_enabled():
        return fn(x, *more)
    out = None
    for lo in range(0, rows, chunk):
        part = fn(*(t[..., lo : lo + chunk, :, :] for t in (x, *more)))
        if out is None:
            out = part.new_empty(*part.shape[:-3], rows, *part.shape[-2:])
        out[..., lo : lo + chunk, :, :] = part
    return out


def map_pair_rows(fn, x, budget: int, bytes_per_position: int, *more):
    return map_row_chunks(fn, x, budget_rows(budget, x.shape[-2], bytes_per_position), *more)


def map_pair_transition(transition, x, budget: int, factor: int):
    return map_pair_rows(transition, x, budget, 2 * factor * x.shape[-1] * gemm_itemsize(x))
