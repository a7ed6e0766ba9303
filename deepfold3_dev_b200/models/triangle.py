"""Triangle multiplicative update (plain and multi-head-routed) and outer-product-mean.

Reference behaviour: model/ops.py:171-785. Semantics kept exactly:
``a`` and ``b`` are the even / odd channels of ``sigmoid(gate(z0)) * proj(z0)``
(interleaved, not halves); outgoing contracts ``a[i,k] b[j,k]``, incoming
``a[k,j] b[k,i]``; the result passes ``norm_center``, ``out_proj`` and the
``sigmoid(out_gate(z0))`` gate.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from .. import ops
from .primitives import LayerNorm, LinearNoBias

_HEAD_NORMS = ("channel", "head_rms", "head_ln", "post_channel")


class _RouterWindow:
    """Running means of router read-outs between two log lines (host floats; one update per routed forward).

    Read-outs of a gain tensor ``g [..., H]``: entropy of the per-position head distribution and of its average over
    positions (both divided by log H, so 1 = uniform), RMS / spread / mean of the gains, and the largest and smallest
    average share of any head.
    """

    def __init__(self, num_heads: int):
        self.h = max(int(num_heads), 1)
        self.count, self.totals = 0, {}

    @torch.no_grad()
    def add(self, gains: torch.Tensor) -> None:
        g = gains.reshape(-1, self.h)
        dist = g / g.sum(dim=-1, keepdim=True).clamp_min(1e-9)
        avg = dist.mean(dim=0)
        norm = math.log(self.h) if self.h > 1 else 1.0
        ent = lambda p: -(p * (p + 1e-9).log()).sum(dim=-1)  # noqa: E731
        sample = {
            "entropy": ent(dist).mean() / norm, "marginal_entropy": ent(avg) / norm, "g_rms": g.square().mean(dim=-1).sqrt().mean(),
            "g_std": g.std(dim=0).mean(), "g_mean": g.mean(), "occupancy_max": avg.max(), "occupancy_min": avg.min(),
        }  # fmt: skip
        for key, value in sample.items():
            self.totals[key] = self.totals.get(key, 0.0) + float(value)
        self.count += 1

    def means(self, reset: bool = True):
        if self.count == 0:
            return None
        out = {key: total / self.count for key, total in self.totals.items()}
        if reset:
            self.count, self.totals = 0, {}
        return out


class _TriangleMulBase(nn.Module):
    outgoing: bool = True

    def __init__(self, c_z, optim=None, num_heads=0, head_norm="channel", router=False, router_kind="softmax"):
        super().__init__()
        if head_norm not in _HEAD_NORMS:
            raise ValueError(f"head_norm must be channel|head_rms|head_ln|post_channel, got {head_norm!r}")
        if head_norm == "post_channel" and not router:
            raise ValueError("head_norm='post_channel' is meaningless without router=True")
        if router_kind not in ("softmax", "sigmoid"):
            raise ValueError(f"router_kind must be softmax|sigmoid, got {router_kind!r}")
        if head_norm != "channel" or router:
            if num_heads <= 0:
                raise ValueError("num_heads > 0 is required for per-head norm or routing")
            if c_z % num_heads:
                raise ValueError(f"c_z={c_z} must be divisible by num_heads={num_heads}")
        self.c_z = c_z
        self.norm_left = LayerNorm(c_z)
        self.proj = LinearNoBias(c_z, c_z * 2)
        self.gate = LinearNoBias(c_z, c_z * 2, initializer="zeros")
        self.norm_center = LayerNorm(c_z, bias=head_norm != "head_rms")
        self.out_proj = LinearNoBias(c_z, c_z, initializer="zeros")
        self.out_gate = LinearNoBias(c_z, c_z, initializer="zeros")
        self.num_heads = int(num_heads)
        self.head_dim = c_z // num_heads if num_heads else 0
        self.head_norm = head_norm
        self.use_router = bool(router)
        self.router_kind = router_kind
        self.is_mhr = head_norm != "channel" or self.use_router
        self.router = LinearNoBias(c_z, num_heads, initializer="zeros") if self.use_router else None
        self.router_stats_enabled = False
        self._router_window = _RouterWindow(self.num_heads)

    # ---- multi-head variants: the contraction result is cut into heads between the contraction and out_proj.
    # Each head may get its own normalisation (instead of one LayerNorm over all channels) and, with a router, a
    # per-position gain predicted from the input (behaviour of the reference's model/ops.py:475-549).
    def _head_gains(self, router_logits):
        """``[..., H]`` gains with mean 1 at initialisation (zero router weights): H * softmax, or 2 * sigmoid."""
        logits = router_logits.float()
        if self.router_kind == "softmax":
            gains = torch.softmax(logits, dim=-1) * float(self.num_heads)
        else:
            gains = torch.sigmoid(logits) * 2.0
        if self.router_stats_enabled:
            self._router_window.add(gains)
        return gains

    def _per_head_norm(self, heads):
        """``heads [..., H, d]`` normalised inside each head in fp32, with norm_center's weight (and bias) cut per head."""
        nc, shape = self.norm_center, (self.num_heads, self.head_dim)
        x = heads.float()
        if self.head_norm == "head_ln":
            x = x - x.mean(dim=-1, keepdim=True)
        x = x * torch.rsqrt(x.square().mean(dim=-1, keepdim=True) + nc.eps)
        x = x.to(heads.dtype) * nc.weight.view(shape)
        return x + nc.bias.view(shape) if self.head_norm == "head_ln" else x

    def _head_mix(self, act, router_logits):
        split = (self.num_heads, self.head_dim)
        gains = None if router_logits is None else self._head_gains(router_logits).to(act.dtype).unsqueeze(-1)
        if self.head_norm == "post_channel":  # route first, one LayerNorm over all channels afterwards
            routed = act.unflatten(-1, split) * gains
            return self.norm_center(routed.flatten(-2))
        heads = self.norm_center(act).unflatten(-1, split) if self.head_norm == "channel" else self._per_head_norm(act.unflatten(-1, split))
        if gains is not None:
            heads = heads * gains
        return heads.flatten(-2)

    def _flush_router_stats(self, reset=True):
        return self._router_window.means(reset)

    def forward(self, z: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        squeeze = z.dim() == 3
        if squeeze:
            z, mask = z.unsqueeze(0), mask.unsqueeze(0)
        z0 = self.norm_left(z)
        router_logits = self.router(z0) if self.use_router else None
        if self.is_mhr:
            act = ops.triangle_projection_contract(z0, self.gate.weight, self.proj.weight, mask, self.outgoing)
            act = self.out_proj(self._head_mix(act, router_logits))
        else:
            nc = self.norm_center
            act = ops.triangle_contract_norm(z0, self.gate.weight, self.proj.weight, mask, self.outgoing, nc.weight, nc.bias, nc.eps)
            if nc.output_scale != 1.0:
                act = act * nc.output_scale
            act = self.out_proj(act)
        out = ops.sigmoid_gate_mul(z0, self.out_gate.weight, act)
        return out.squeeze(0) if squeeze else out


class TriangleMulOutgoing(_TriangleMulBase):
    outgoing = True


class TriangleMulIncoming(_TriangleMulBase):
    outgoing = False


def _routed_modules(model: nn.Module):
    return [(name, m) for name, m in model.named_modules() if isinstance(m, _TriangleMulBase) and m.use_router]


def set_router_stats_enabled(model: nn.Module, enabled: bool) -> None:
    """Switch the router read-outs of every routed triangle multiply on or off (they cost a few host reads per forward)."""
    for _, module in _routed_modules(model):
        module.router_stats_enabled = bool(enabled)


# (log key, read-out, how to combine the per-module window means)
_ROUTER_SUMMARY = (
    ("entropy", "entropy", "mean"), ("entropy_min", "entropy", "min"), ("marginal_entropy", "marginal_entropy", "mean"),
    ("g_std", "g_std", "mean"), ("g_std_max", "g_std", "max"), ("g_mean", "g_mean", "mean"), ("g_rms", "g_rms", "mean"),
    ("g_rms_max", "g_rms", "max"), ("occupancy_max", "occupancy_max", "max"), ("occupancy_min", "occupancy_min", "min"),
)  # fmt: skip
_COMBINE = {"mean": lambda xs: sum(xs) / len(xs), "min": min, "max": max}


def collect_router_stats(model: nn.Module, prefix: str = "router", reset: bool = True) -> dict[str, float]:
    """Log entries for the routed triangle multiplies: their window means combined over modules (mean, and worst case
    where that is the interesting one), the gap between marginal and per-position entropy (how much heads specialise by
    position), and four read-outs per module (reference: model/ops.py:110-170)."""
    per_module = {name: m._flush_router_stats(reset) for name, m in _routed_modules(model)}
    per_module = {name: r for name, r in per_module.items() if r is not None}
    if not per_module:
        return {}
    rows = list(per_module.values())
    out = {f"{prefix}/{key}": _COMBINE[how]([r[field] for r in rows]) for key, field, how in _ROUTER_SUMMARY}
    out[f"{prefix}/specialization_gap"] = _COMBINE["mean"]([r["marginal_entropy"] - r["entropy"] for r in rows])
    for name, r in per_module.items():
        out.update({f"{prefix}/{field}_by_module/{name}": r[field] for field in ("entropy", "marginal_entropy", "g_rms", "g_std")})
    return out


class OuterProductMean(nn.Module):
    """MSA → pair update (reference: ops.py:683-785)."""

    def __init__(self, c_msa: int, c_z: int, c_hidden: int = 32):
        super().__init__()
        self.norm = LayerNorm(c_msa)
        self.proj_a = LinearNoBias(c_msa, c_hidden)
        self.proj_b = LinearNoBias(c_msa, c_hidden)
        self.out_w = nn.Parameter(torch.zeros(c_hidden, c_hidden, c_z))
        self.out_b = nn.Parameter(torch.zeros(c_z))
        self._chunk_size = 0
        self._row_chunk = 0

    def forward(self, msa: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        squeeze = msa.dim() == 3
        if squeeze:
            msa, mask = msa.unsqueeze(0), mask.unsqueeze(0)
        m = mask.unsqueeze(-1)
        x = self.norm(msa)
        a = self.proj_a(x) * m.to(x.dtype)
        b = self.proj_b(x) * m.to(x.dtype)
        N, chunk = a.shape[2], self._chunk_size
        if 0 < chunk < N and not torch.is_grad_enabled():
            out = a.new_empty(a.shape[0], N, N, self.out_w.shape[2])
            for i0 in range(0, N, chunk):
                for j0 in range(0, N, chunk):
                    out[:, i0 : i0 + chunk, j0 : j0 + chunk] = ops.outer_product_mean(
                        a[:, :, i0 : i0 + chunk], b[:, :, j0 : j0 + chunk], self.out_w, self.out_b,
                        None, mask_i=mask[:, :, i0 : i0 + chunk], mask_j=mask[:, :, j0 : j0 + chunk],
                    )  # fmt: skip
        else:
            out = ops.outer_product_mean(a, b, self.out_w, self.out_b, mask)
        return out.squeeze(0) if squeeze else out
