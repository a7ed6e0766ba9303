"""Masked-MSA (BERT) corruption and prediction head (reference: model/masked_msa.py:33-223)."""

from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .primitives import LayerNorm, LinearNoBias, af3_linear_init_

MSA_VOCAB_SIZE = 32
MSA_MASK = 31


def _masked_softmax(logits, mask, dim):
    """fp32 softmax over valid positions; a fully masked row gives all-zero weights."""
    logits = logits.float()
    mask = mask.bool()
    probs = logits.masked_fill(~mask, torch.finfo(logits.dtype).min).softmax(dim=dim)
    probs = torch.where(mask, probs, torch.zeros_like(probs))
    return probs / probs.sum(dim=dim, keepdim=True).clamp_min(1e-8)


@torch.no_grad()
def apply_bert_mask(msa, msa_mask, profile, cfg, generator=None):
    """Corrupt ``replace_fraction`` of valid MSA entries.

    The replacement of an entry is drawn from ``uniform_prob * U(20 amino acids)
    + profile_prob * profile + same_prob * one_hot(entry)`` with the remaining
    mass on the mask token. Returns ``(corrupted, original, corrupted_flag)``.
    """
    V, dev = MSA_VOCAB_SIZE, msa.device
    uniform = torch.zeros(V, device=dev)
    uniform[:20] = 0.05
    probs = cfg.same_prob * F.one_hot(msa.long(), V).float() + cfg.uniform_prob * uniform
    if profile is not None and cfg.profile_prob > 0.0:
        prof = profile.float()
        prof = F.pad(prof, (0, V - prof.shape[-1])) if prof.shape[-1] < V else prof[..., :V]
        probs = probs + cfg.profile_prob * prof.unsqueeze(-3)
    probs = probs.clone()
    probs[..., MSA_MASK] += 1.0 - cfg.uniform_prob - cfg.profile_prob - cfg.same_prob
    flat = probs.reshape(-1, V).clamp_min(0.0)
    flat = flat / flat.sum(dim=-1, keepdim=True).clamp_min(1e-8)
    drawn = torch.multinomial(flat, 1, generator=generator).reshape(msa.shape)
    hit = (torch.rand(msa.shape, device=dev, generator=generator) < cfg.replace_fraction) & msa_mask.bool()
    return torch.where(hit, drawn.to(msa.dtype), msa), msa.clone(), hit.to(torch.float32)


class MaskedMSAHead(nn.Module):
    """Each token's single vector attends over its MSA column; an MLP on ``[msa, single, context]`` gives logits."""

    def __init__(self, cfg, c_msa: int, c_single: int):
        super().__init__()
        self.cfg = cfg
        self.num_heads, self.head_dim = int(cfg.num_heads), int(cfg.head_dim)
        d = self.num_heads * self.head_dim
        self._attn_scale = 1.0 / math.sqrt(self.head_dim)
        self.msa_norm = LayerNorm(c_msa)
        self.single_norm = LayerNorm(c_single)
        self.q_proj = LinearNoBias(c_single, d)
        self.k_proj = LinearNoBias(c_msa, d)
        self.v_proj = LinearNoBias(c_msa, d)
        self.mlp1 = LinearNoBias(c_msa + c_single + d, cfg.hidden_dim, initializer="relu")
        self.mlp2 = LinearNoBias(cfg.hidden_dim, cfg.hidden_dim, initializer="relu")
        self.out = nn.Linear(cfg.hidden_dim, cfg.c_out, bias=cfg.out_bias)
        af3_linear_init_(self.out.weight, "linear")
        if cfg.out_bias:
            nn.init.zeros_(self.out.bias)

    def forward(self, msa, single, msa_mask=None):
        m, s = self.msa_norm(msa), self.single_norm(single)
        H, D = self.num_heads, self.head_dim
        q = self.q_proj(s).unflatten(-1, (H, D))
        k = self.k_proj(m).unflatten(-1, (H, D))
        v = self.v_proj(m).unflatten(-1, (H, D))
        att = torch.einsum("...nhd,...snhd->...nhs", q, k) * self._attn_scale
        if msa_mask is not None:
            att = _masked_softmax(att, msa_mask.bool().transpose(-1, -2).unsqueeze(-2), dim=-1).to(v.dtype)
        else:
            att = att.float().softmax(dim=-1).to(v.dtype)
        ctx = torch.einsum("...nhs,...snhd->...nhd", att, v).flatten(-2)
        # first MLP layer applied to the three concatenated parts separately, so the
        # [S, N, c_msa + c_single + d] concatenation is never formed
        cm, cs = m.shape[-1], s.shape[-1]
        w1 = self.mlp1.weight
        per_token = F.linear(s, w1[:, cm : cm + cs]) + F.linear(ctx, w1[:, cm + cs :])
        x = F.relu(F.linear(m, w1[:, :cm]) + per_token.unsqueeze(-3))
        return self.out(F.relu(self.mlp2(x)))
