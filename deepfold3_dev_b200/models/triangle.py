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
        self._router_stats = None

    # ---- multi-head routing between contraction and out_proj (reference: ops.py:475-549) ----
    def _route(self, t, router_logits):
        if router_logits is None:
            return t
        r = router_logits.float()
        h = self.num_heads
        g = float(h) * torch.softmax(r, dim=-1) if self.router_kind == "softmax" else 2.0 * torch.sigmoid(r)
        if self.router_stats_enabled:
            self._record_router_stats(g)
        return t * g.to(t.dtype).unsqueeze(-1)

    def _head_mix(self, act, router_logits):
        h, d = self.num_heads, self.head_dim
        if self.head_norm == "post_channel":
            return self.norm_center(self._route(act.unflatten(-1, (h, d)), router_logits).flatten(-2))
        if self.head_norm == "channel":
            t = self.norm_center(act).unflatten(-1, (h, d))
        else:
            t32 = act.unflatten(-1, (h, d)).float()
            w = self.norm_center.weight.view(h, d)
            eps = self.norm_center.eps
            if self.head_norm == "head_rms":
                t = (t32 * torch.rsqrt(t32.pow(2).mean(-1, keepdim=True) + eps)).to(act.dtype) * w
            else:
                mu = t32.mean(-1, keepdim=True)
                t32 = (t32 - mu) * torch.rsqrt(t32.var(-1, keepdim=True, unbiased=False) + eps)
                t = t32.to(act.dtype) * w + self.norm_center.bias.view(h, d)
        return self._route(t, router_logits).flatten(-2)

    @torch.no_grad()
    def _record_router_stats(self, g):
        H = self.num_heads
        g = g.reshape(-1, H)
        p = g / g.sum(-1, keepdim=True).clamp_min(1e-9)
        share = p.mean(0)
        vals = dict(
            entropy=float(-(p * (p + 1e-9).log()).sum(-1).mean() / math.log(H)),
            marginal_entropy=float(-(share * (share + 1e-9).log()).sum() / math.log(H)),
            g_rms=float(g.pow(2).mean(-1).sqrt().mean()),
            g_std=float(g.std(0).mean()),
            g_mean=float(g.mean()),
            occupancy_max=float(share.max()),
            occupancy_min=float(share.min()),
            n=1.0,
        )
        if self._router_stats is None:
            self._router_stats = {k: 0.0 for k in vals}
        for k, v in vals.items():
            self._router_stats[k] += v

    def _flush_router_stats(self, reset=True):
        acc = self._router_stats
        if acc is None or acc["n"] == 0:
            return None
        out = {k: v / acc["n"] for k, v in acc.items() if k != "n"}
        if reset:
            self._router_stats = None
        return out

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


def set_router_stats_enabled(model: nn.Module, enabled: bool) -> None:
    for mod in model.modules():
        if isinstance(mod, _TriangleMulBase) and mod.use_router:
            mod.router_stats_enabled = bool(enabled)


def collect_router_stats(model: nn.Module, prefix: str = "router", reset: bool = True) -> dict[str, float]:
    """Window means of the router read-outs over all routed triangle multiplies (reference: ops.py:117-168)."""
    rows = []
    for name, mod in model.named_modules():
        if isinstance(mod, _TriangleMulBase) and mod.use_router:
            r = mod._flush_router_stats(reset)
            if r is not None:
                rows.append((name, r))
    if not rows:
        return {}
    n = len(rows)
    mean = lambda k: sum(r[k] for _, r in rows) / n  # noqa: E731
    out = {
        f"{prefix}/entropy": mean("entropy"),
        f"{prefix}/entropy_min": min(r["entropy"] for _, r in rows),
        f"{prefix}/marginal_entropy": mean("marginal_entropy"),
        f"{prefix}/specialization_gap": sum(r["marginal_entropy"] - r["entropy"] for _, r in rows) / n,
        f"{prefix}/g_std": mean("g_std"),
        f"{prefix}/g_std_max": max(r["g_std"] for _, r in rows),
        f"{prefix}/g_mean": mean("g_mean"),
        f"{prefix}/occupancy_max": max(r["occupancy_max"] for _, r in rows),
        f"{prefix}/occupancy_min": min(r["occupancy_min"] for _, r in rows),
        f"{prefix}/g_rms": mean("g_rms"),
        f"{prefix}/g_rms_max": max(r["g_rms"] for _, r in rows),
    }
    for name, r in rows:
        for k in ("entropy", "marginal_entropy", "g_rms", "g_std"):
            out[f"{prefix}/{k}_by_module/{name}"] = r[k]
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
