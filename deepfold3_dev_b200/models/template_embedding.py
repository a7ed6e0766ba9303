"""Template embedding: per-template pair features → 2 pair-only blocks at c=64 → average → pair update.

Reference: model/template_embedding.py:67-570. State-dict names
(``single_template_emb.embed_*``, ``pairformer.{i}``, ``output_proj``) match.
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from .attention import GridSelfAttention
from .embedders import dgram_from_positions
from .primitives import Gain as _gain
from .primitives import (
    LayerNorm,
    LinearNoBias,
    block_residual_scale,
    make_transition_block,
    map_pair_rows,
    map_pair_transition,
)
from .triangle import TriangleMulIncoming, TriangleMulOutgoing

_CA_IDX, _CB_IDX, _GLY_IDX = 1, 3, 7


def pseudo_beta_from_positions(aatype, positions, mask):
    """CB position and mask per residue, CA for glycine (dense-atom slots CA=1, CB=3)."""
    gly = aatype == _GLY_IDX
    pos = torch.where(gly.unsqueeze(-1), positions[:, _CA_IDX], positions[:, _CB_IDX])
    return pos, torch.where(gly, mask[:, _CA_IDX], mask[:, _CB_IDX])


def unit_vectors_in_frames(frames, origins, frame_mask, eps: float = 1e-8):
    """Unit displacement ``origin_j - origin_i`` expressed in residue ``i``'s frame (fp32).

    ``frames``: ``[..., N, 3, 3]`` with rows the local axes. Returns
    ``(unit [..., N, N, 3], mask2d [..., N, N])``.
    """
    f32, o32 = frames.float(), origins.float()
    disp = o32.unsqueeze(-2) - o32.unsqueeze(-3)
    local = torch.einsum("...iae,...ije->...ija", f32, disp)
    unit = local / local.norm(dim=-1, keepdim=True).clamp(min=eps)
    mask2d = frame_mask.unsqueeze(-1) * frame_mask.unsqueeze(-2)
    return (unit * mask2d.unsqueeze(-1).float()).to(origins.dtype), mask2d


class TemplatePairFormerBlock(nn.Module):
    """Pair-only block: triangle multiplications, row/column attention, transition."""

    def __init__(self, num_channels, num_heads=4, num_intermediate_factor=2, pair_dropout=0.25, optim=None,
                 residual_out_scale=1.0):  # fmt: skip
        super().__init__()
        self.tri_mul_out = TriangleMulOutgoing(num_channels, optim=optim)
        self.tri_mul_in = TriangleMulIncoming(num_channels, optim=optim)
        self.pair_attn_row = GridSelfAttention(num_channels, num_heads=num_heads, transpose=False, optim=optim)
        self.pair_attn_col = GridSelfAttention(num_channels, num_heads=num_heads, transpose=True, optim=optim)
        self.pair_transition = make_transition_block(num_channels, num_intermediate_factor, config=optim)
        self.num_intermediate_factor = num_intermediate_factor
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.pair_dropout = pair_dropout
        self.residual_out_scale = float(residual_out_scale)

    def forward(self, pair, pair_mask):
        p, tr, s = self.pair_dropout, self.training, self.residual_out_scale
        pair = ops.dropout_add(pair, _gain(s) * self.tri_mul_out(pair, pair_mask), p, tr, -3)
        pair = ops.dropout_add(pair, _gain(s) * self.tri_mul_in(pair, pair_mask), p, tr, -3)
        pair = ops.dropout_add(pair, _gain(s) * self.pair_attn_row(pair, pair_mask), p, tr, -3)
        pair = ops.dropout_add(pair, _gain(s) * self.pair_attn_col(pair, pair_mask), p, tr, -2)
        return pair + _gain(s) * map_pair_transition(
            self.pair_transition, pair, self.pair_chunk_budget, self.num_intermediate_factor
        )


class SingleTemplateEmbedding(nn.Module):
    """Nine projected template features summed, refined by the pair-only stack, then normalised."""

    def __init__(self, cfg, optim=None):
        super().__init__()
        c, pc = cfg.num_channels, cfg.pair_channel
        self.cfg = cfg
        self._grad_checkpoint = bool(optim and optim.use_gradient_checkpointing)
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.embed_dgram = LinearNoBias(cfg.dgram_num_bins, c, initializer="relu")
        self.embed_pseudo_beta = LinearNoBias(1, c, initializer="relu")
        self.embed_aatype_row = LinearNoBias(cfg.aatype_num_classes, c, initializer="relu")
        self.embed_aatype_col = LinearNoBias(cfg.aatype_num_classes, c, initializer="relu")
        self.embed_unit_vec_x = LinearNoBias(1, c, initializer="relu")
        self.embed_unit_vec_y = LinearNoBias(1, c, initializer="relu")
        self.embed_unit_vec_z = LinearNoBias(1, c, initializer="relu")
        self.embed_backbone_mask = LinearNoBias(1, c, initializer="relu")
        self.embed_query = LinearNoBias(pc, c, initializer="relu")
        self.query_norm = LayerNorm(pc)
        pf = cfg.pairformer
        self.pairformer = nn.ModuleList(
            TemplatePairFormerBlock(
                pf.num_channels, pf.num_heads, pf.num_intermediate_factor, pf.pair_dropout, optim,
                block_residual_scale(i, pf.num_layer, pf.residual_output_scaling, pf.uniform_residual_scale),
            )  # fmt: skip
            for i in range(pf.num_layer)
        )
        self.output_norm = LayerNorm(c)

    def forward(self, query_pair, template_aatype, template_pseudo_beta, template_pseudo_beta_mask,
                template_backbone_frame, template_backbone_mask, pair_mask, multichain_mask=None,
                template_ca=None):  # fmt: skip
        dtype = query_pair.dtype
        cfg = self.cfg
        pb_mask2d = template_pseudo_beta_mask.unsqueeze(-1) * template_pseudo_beta_mask.unsqueeze(-2)
        if multichain_mask is not None:
            pb_mask2d = pb_mask2d * multichain_mask
        dgram = dgram_from_positions(
            template_pseudo_beta, cfg.dgram_min_bin, cfg.dgram_max_bin, self.embed_dgram.in_features
        ) * pb_mask2d.unsqueeze(-1)
        points = template_ca if template_ca is not None else template_pseudo_beta
        unit, bb_mask2d = unit_vectors_in_frames(template_backbone_frame, points, template_backbone_mask)
        if multichain_mask is not None:
            bb_mask2d = bb_mask2d * multichain_mask
        unit = unit * bb_mask2d.unsqueeze(-1).to(unit.dtype)

        aa = F.one_hot(template_aatype, self.embed_aatype_row.in_features).to(dtype)
        act = self.embed_dgram(dgram.to(dtype))
        act = act + self.embed_pseudo_beta(pb_mask2d.unsqueeze(-1).to(dtype))
        # one-hot(aatype) @ W broadcast over the other axis: row term varies with j, column term with i
        act = act + self.embed_aatype_row(aa).unsqueeze(-3) + self.embed_aatype_col(aa).unsqueeze(-2)
        act = act + self.embed_unit_vec_x(unit[..., 0:1].to(dtype))
        act = act + self.embed_unit_vec_y(unit[..., 1:2].to(dtype))
        act = act + self.embed_unit_vec_z(unit[..., 2:3].to(dtype))
        act = act + self.embed_backbone_mask(bb_mask2d.unsqueeze(-1).to(dtype))
        act = act + map_pair_rows(
            lambda rows: self.embed_query(self.query_norm(rows)), query_pair, self.pair_chunk_budget,
            4 * query_pair.shape[-1],
        )  # fmt: skip
        use_ckpt = self._grad_checkpoint and torch.is_grad_enabled()
        for layer in self.pairformer:
            if use_ckpt:
                act = checkpoint(layer, act, pair_mask, use_reentrant=False, determinism_check="none")
            else:
                act = layer(act, pair_mask)
        return self.output_norm(act)


class TemplateEmbedding(nn.Module):
    """Average of the per-template embeddings over real template slots, ReLU, project to the pair width."""

    def __init__(self, cfg, optim=None):
        super().__init__()
        self.cfg = cfg
        self.single_template_emb = SingleTemplateEmbedding(cfg, optim=optim)
        self.output_proj = LinearNoBias(cfg.num_channels, cfg.pair_channel, initializer="relu")

    def forward(self, query_pair, template_aatype, template_pseudo_beta, template_pseudo_beta_mask,
                template_backbone_frame, template_backbone_mask, pair_mask, multichain_mask=None,
                template_ca=None, template_mask=None):  # fmt: skip
        batched = query_pair.dim() == 4
        t_axis = 1 if batched else 0
        T = template_aatype.shape[t_axis]
        dtype = query_pair.dtype
        if template_mask is not None:
            template_mask = template_mask.to(dtype)
        summed = query_pair.new_zeros(*query_pair.shape[:-1], self.cfg.num_channels)
        pick = (lambda x, t: x[:, t]) if batched else (lambda x, t: x[t])
        for t in range(T):
            emb = self.single_template_emb(
                query_pair,
                pick(template_aatype, t),
                pick(template_pseudo_beta, t),
                pick(template_pseudo_beta_mask, t),
                pick(template_backbone_frame, t),
                pick(template_backbone_mask, t),
                pair_mask,
                multichain_mask,
                pick(template_ca, t) if template_ca is not None else None,
            )
            if template_mask is None:
                summed = summed + emb
            else:
                m = pick(template_mask, t)
                summed = torch.addcmul(summed, emb, m.view(-1, 1, 1, 1) if batched else m)
        if template_mask is None:
            avg = summed / (T + 1e-7)
        else:
            n_real = template_mask.sum(dim=-1)
            avg = summed / ((n_real.view(-1, 1, 1, 1) if batched else n_real) + 1e-7)
        return self.output_proj(F.relu(avg))
