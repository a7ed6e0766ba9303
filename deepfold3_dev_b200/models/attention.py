"""Attention modules: triangle (grid) attention, MSA row attention, single attention.

Parameter names follow the reference (model/attention.py:56-452). All three
accept inputs with or without a leading batch axis. The softmax-attention core
is ``ops.pair_bias_attention`` over the layout ``[B, R, H, N, D]`` with a bias
``[B, H, N, N]`` shared across the ``R`` independent rows.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .primitives import LayerNorm, LinearNoBias, biased_linear, map_pair_rows, map_row_chunks


class GridSelfAttention(nn.Module):
    """Gated self-attention along the rows (``transpose=False``) or columns of the pair tensor.

    Row attention: for every row ``r`` softmax over ``j`` of
    ``q[r,i]·k[r,j]/sqrt(D) + bias[h,i,j] + mask``. Column attention does the
    same along rows for each column; both use the bias indexed by
    (query token, key token) (reference: attention.py:167-269).
    """

    def __init__(self, c: int, num_heads: int = 4, transpose: bool = False, optim=None):
        super().__init__()
        assert c % num_heads == 0
        self.num_heads = num_heads
        self.head_dim = max(c // num_heads, 16)
        self.transpose = transpose
        self.scale = self.head_dim**-0.5
        hd = num_heads * self.head_dim
        self.norm = LayerNorm(c)
        self.pair_bias = LinearNoBias(c, num_heads)
        self.to_q = LinearNoBias(c, hd)
        self.to_k = LinearNoBias(c, hd)
        self.to_v = LinearNoBias(c, hd)
        self.to_g = LinearNoBias(c, hd, initializer="zeros")
        self.out_proj = LinearNoBias(hd, c, initializer="zeros")

    def forward(self, z: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        squeeze = z.dim() == 3
        if squeeze:
            z, mask = z.unsqueeze(0), mask.unsqueeze(0)
        B, N, _, C = z.shape
        H, D = self.num_heads, self.head_dim

        zn = self.norm(z)
        bias = ops.head_bias_planes(zn, self.pair_bias.weight)  # [B, H, N, N] (query, key)
        qkv = ops.stacked_linear(zn, self.to_q.weight, self.to_k.weight, self.to_v.weight).view(B, N, N, 3, H, D)

        key_mask = mask.transpose(1, 2) if self.transpose else mask
        out = ops.grid_attention(qkv, bias, key_mask, self.scale, self.transpose)
        out = out.permute(0, 3, 1, 2, 4) if self.transpose else out.permute(0, 1, 3, 2, 4)
        out = out.reshape(B, N, N, H * D)
        out = self.out_proj(ops.sigmoid_gate_mul(zn, self.to_g.weight, out))
        return out.squeeze(0) if squeeze else out


class MSAAttention(nn.Module):
    """MSA row update weighted by pair-derived attention (reference: attention.py:272-341).

    The weights ``softmax_k(W LN(pair))`` are computed once and shared by all
    MSA rows; the update is a weighted average of ``to_v(LN(msa))`` over keys.
    """

    def __init__(self, c_msa: int, c_pair: int, num_heads: int = 8, optim=None):
        super().__init__()
        assert c_msa % num_heads == 0
        self.num_heads = num_heads
        self.head_dim = c_msa // num_heads
        hd = num_heads * self.head_dim
        self.norm = LayerNorm(c_msa)
        self.pair_norm = LayerNorm(c_pair)
        self.pair_logits = LinearNoBias(c_pair, num_heads)
        self.to_v = LinearNoBias(c_msa, hd)
        self.to_g = LinearNoBias(c_msa, hd, initializer="zeros")
        self.out_proj = LinearNoBias(hd, c_msa, initializer="zeros")
        self.row_chunk = optim.msa_row_chunk if optim is not None else 0
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0

    def _weights(self, mask, pair):
        logits = map_pair_rows(
            lambda rows: self.pair_logits(self.pair_norm(rows)), pair, self.pair_chunk_budget, 4 * pair.shape[-1]
        ).permute(0, 3, 1, 2)
        col_mask = mask.max(dim=-2).values
        logits = logits.float() + 1e9 * (col_mask.float() - 1.0)[:, None, None, :]
        return F.softmax(logits, dim=-1)

    def _rows(self, msa, w):
        B, S, N, _ = msa.shape
        H, D = self.num_heads, self.head_dim
        m = self.norm(msa)
        v = self.to_v(m).view(B, S, N, H, D)
        avg = ops.msa_weighted_average(w.to(v.dtype), v).reshape(B, S, N, H * D)
        return self.out_proj(avg * torch.sigmoid(self.to_g(m)))

    def forward(self, msa, mask, pair):
        squeeze = msa.dim() == 3
        if squeeze:
            msa, mask, pair = msa.unsqueeze(0), mask.unsqueeze(0), pair.unsqueeze(0)
        w = self._weights(mask, pair)
        out = map_row_chunks(lambda rows: self._rows(rows, w), msa, self.row_chunk)
        return out.squeeze(0) if squeeze else out


class SingleAttention(nn.Module):
    """Pair-biased self-attention over the single representation (reference: attention.py:344-452)."""

    def __init__(
        self,
        c: int,
        num_heads: int = 16,
        key_dim: int = 384,
        value_dim: int = 384,
        optim=None,
        pair_bias_gate: bool = False,
        pair_bias_gate_init_tau: float = 0.25,
    ):
        super().__init__()
        assert key_dim % num_heads == 0 and value_dim % num_heads == 0
        self.num_heads = num_heads
        self.key_dim_per_head = key_dim // num_heads
        self.val_dim_per_head = value_dim // num_heads
        self.scale = self.key_dim_per_head**-0.5
        self.norm = LayerNorm(c)
        if pair_bias_gate:
            if pair_bias_gate_init_tau <= 0.0:
                raise ValueError(f"pair_bias_gate_init_tau must be > 0, got {pair_bias_gate_init_tau}")
            self.pair_bias_gate_a = nn.Parameter(torch.full((num_heads,), math.log(float(pair_bias_gate_init_tau))))
        else:
            self.register_parameter("pair_bias_gate_a", None)
        self.to_q = biased_linear(c, key_dim, "linear")
        self.to_k = LinearNoBias(c, key_dim)
        self.to_v = LinearNoBias(c, value_dim)
        self.to_g = LinearNoBias(c, value_dim, initializer="zeros")
        self.out_proj = LinearNoBias(value_dim, c, initializer="zeros")

    def forward(self, x, mask, pair_logits):
        squeeze = x.dim() == 2
        if squeeze:
            x, mask, pair_logits = x.unsqueeze(0), mask.unsqueeze(0), pair_logits.unsqueeze(0)
        B, N, _ = x.shape
        H, Dk, Dv = self.num_heads, self.key_dim_per_head, self.val_dim_per_head
        xn = self.norm(x)
        q = self.to_q(xn).view(B, 1, N, H, Dk).permute(0, 1, 3, 2, 4)
        k = self.to_k(xn).view(B, 1, N, H, Dk).permute(0, 1, 3, 2, 4)
        v = self.to_v(xn).view(B, 1, N, H, Dv).permute(0, 1, 3, 2, 4)
        if self.pair_bias_gate_a is not None:
            pair_logits = pair_logits * torch.exp(self.pair_bias_gate_a).to(pair_logits.dtype).view(1, H, 1, 1)
        out = ops.pair_bias_attention(q, k, v, pair_logits, mask.view(B, 1, N), self.scale)
        out = out.permute(0, 1, 3, 2, 4).reshape(B, N, H * Dv)
        out = self.out_proj(out * torch.sigmoid(self.to_g(xn)))
        return out.squeeze(0) if squeeze else out
