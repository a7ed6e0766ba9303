"""Trunk: input embeddings, 4-block MSA stack, 48-block Pairformer.

Reference: model/evoformer.py:100-608. Sub-module order inside each block and
the dropout sharing (rows for everything except column attention) are kept.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops
from .attention import GridSelfAttention, MSAAttention, SingleAttention
from .branch_scaler import make_branch_scaler
from .primitives import Gain as _gain
from .primitives import (
    LayerNorm,
    LinearNoBias,
    block_residual_scale,
    budget_rows,
    make_transition_block,
    map_pair_rows,
    map_pair_transition,
    map_row_chunks,
)
from .template_embedding import TemplateEmbedding
from .triangle import OuterProductMean, TriangleMulIncoming, TriangleMulOutgoing

TARGET_FEAT_DIM = 447  # 63 raw token features + 384 from the atom conditioning encoder
MSA_FEAT_DIM = 34  # one-hot(32) + has_deletion + deletion_value


def _ckpt(fn, *args):
    return checkpoint(fn, *args, use_reentrant=False, determinism_check="none")


def resolve_branch_residual_gain(layer_idx: int, base_gain, per_layer_extra: bool):
    """Extra multiplier of a transition branch; ``None`` when neither knob is set (reference: evoformer.py:66-82)."""
    if base_gain is None and not per_layer_extra:
        return None
    gain = 1.0 if base_gain is None else float(base_gain)
    return gain / math.sqrt(layer_idx + 1.0) if per_layer_extra else gain


def trimul_kwargs(cfg) -> dict:
    return dict(num_heads=cfg.trimul_num_heads, head_norm=cfg.trimul_head_norm, router=cfg.trimul_router,
                router_kind=cfg.trimul_router_kind)  # fmt: skip


class EvoformerBlock(nn.Module):
    """One MSA-stack layer: OPM → MSA row attention → MSA transition → pair updates."""

    def __init__(self, c_msa, c_pair, num_msa_heads=8, num_pair_heads=4, outer_product_hidden=32, msa_dropout=0.15,
                 pair_dropout=0.25, optim=None, residual_out_scale=1.0, use_triangle_attention=True,
                 trimul_kwargs=None):  # fmt: skip
        super().__init__()
        tk = trimul_kwargs or {}
        self.row_attn = MSAAttention(c_msa, c_pair, num_heads=num_msa_heads, optim=optim)
        self.outer_product = OuterProductMean(c_msa, c_pair, c_hidden=outer_product_hidden)
        if optim is not None and optim.tiled_opm_chunk > 0:
            self.outer_product._chunk_size = optim.tiled_opm_chunk
        self.msa_row_chunk = optim.msa_row_chunk if optim is not None else 0
        self.outer_product._row_chunk = self.msa_row_chunk
        self.tri_mul_out = TriangleMulOutgoing(c_pair, optim=optim, **tk)
        self.tri_mul_in = TriangleMulIncoming(c_pair, optim=optim, **tk)
        self.use_triangle_attention = bool(use_triangle_attention)
        if self.use_triangle_attention:
            self.pair_attn_row = GridSelfAttention(c_pair, num_heads=num_pair_heads, transpose=False, optim=optim)
            self.pair_attn_col = GridSelfAttention(c_pair, num_heads=num_pair_heads, transpose=True, optim=optim)
        self.pair_transition = make_transition_block(c_pair, config=optim)
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.msa_transition = make_transition_block(c_msa, config=optim)
        self.msa_dropout = msa_dropout
        self.pair_dropout = pair_dropout
        self.residual_out_scale = float(residual_out_scale)

    def forward(self, msa, pair, msa_mask, pair_mask):
        pp, pm, tr, s = self.pair_dropout, self.msa_dropout, self.training, self.residual_out_scale
        pair = pair + _gain(s) * self.outer_product(msa, msa_mask)
        msa = ops.dropout_add(msa, _gain(s) * self.row_attn(msa, msa_mask, pair), pm, tr, -3)
        msa = msa + _gain(s) * map_row_chunks(self.msa_transition, msa, self.msa_row_chunk)
        pair = ops.dropout_add(pair, _gain(s) * self.tri_mul_out(pair, pair_mask), pp, tr, -3)
        pair = ops.dropout_add(pair, _gain(s) * self.tri_mul_in(pair, pair_mask), pp, tr, -3)
        if self.use_triangle_attention:
            pair = ops.dropout_add(pair, _gain(s) * self.pair_attn_row(pair, pair_mask), pp, tr, -3)
            pair = ops.dropout_add(pair, _gain(s) * self.pair_attn_col(pair, pair_mask), pp, tr, -2)
        pair = pair + _gain(s) * map_pair_transition(self.pair_transition, pair, self.pair_chunk_budget, 4)
        return msa, pair


class PairFormerBlock(nn.Module):
    """One Pairformer layer with the single track (reference: evoformer.py:178-355)."""

    def __init__(self, c_pair, c_single, num_pair_heads=4, num_single_heads=16, single_key_dim=384,
                 single_value_dim=384, pair_dropout=0.25, optim=None, residual_out_scale=1.0, pair_bias_gate=False,
                 pair_bias_gate_init_tau=0.25, single_transition_linear_out_init_gain=None,
                 single_transition_residual_gain=None, pair_transition_residual_gain=None,
                 branch_scaler="identity", use_triangle_attention=True, use_single_track=True,
                 trimul_kwargs=None):  # fmt: skip
        super().__init__()
        tk = trimul_kwargs or {}
        self.tri_mul_out = TriangleMulOutgoing(c_pair, optim=optim, **tk)
        self.tri_mul_in = TriangleMulIncoming(c_pair, optim=optim, **tk)
        self.use_triangle_attention = bool(use_triangle_attention)
        if self.use_triangle_attention:
            self.pair_attn_row = GridSelfAttention(c_pair, num_heads=num_pair_heads, transpose=False, optim=optim)
            self.pair_attn_col = GridSelfAttention(c_pair, num_heads=num_pair_heads, transpose=True, optim=optim)
        self.pair_transition = make_transition_block(c_pair, config=optim)
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.use_single_track = bool(use_single_track)
        if self.use_single_track:
            self.single_to_pair_norm = LayerNorm(c_pair)
            self.single_to_pair = LinearNoBias(c_pair, num_single_heads)
            self.single_attn = SingleAttention(
                c_single, num_heads=num_single_heads, key_dim=single_key_dim, value_dim=single_value_dim, optim=optim,
                pair_bias_gate=pair_bias_gate, pair_bias_gate_init_tau=pair_bias_gate_init_tau,
            )  # fmt: skip
            self.single_transition = make_transition_block(
                c_single, config=optim, linear_out_init_gain=single_transition_linear_out_init_gain
            )
        self.residual_out_scale = float(residual_out_scale)
        self.single_transition_residual_gain = (
            1.0 if single_transition_residual_gain is None else float(single_transition_residual_gain)
        )
        self.pair_transition_residual_gain = (
            1.0 if pair_transition_residual_gain is None else float(pair_transition_residual_gain)
        )
        self.branch_scaler_kind = str(branch_scaler)
        self.branch_scaler = make_branch_scaler(self.branch_scaler_kind)
        self.pair_dropout = pair_dropout

    def _single_bias(self, pair):
        """Pair bias of the single-track attention as contiguous head planes ``[B?, H, N, N]`` (the projection writes
        them channel-major; row chunks under the inference byte budget)."""
        lead = pair.dim() == 3
        z = pair[None] if lead else pair
        N = z.shape[1]
        rows = 0 if torch.is_grad_enabled() else budget_rows(self.pair_chunk_budget, z.shape[-2], 4 * z.shape[-1])
        parts = [ops.head_bias_planes(self.single_to_pair_norm(z[:, lo : lo + (rows or N)]), self.single_to_pair.weight)
                 for lo in range(0, N, rows or N)]  # fmt: skip
        logits = parts[0] if len(parts) == 1 else torch.cat(parts, dim=2)
        return logits[0] if lead else logits

    def forward(self, pair, single, pair_mask, seq_mask):
        p, tr, s = self.pair_dropout, self.training, self.residual_out_scale
        s_pf = _gain(s) * self.pair_transition_residual_gain
        s_sf = _gain(s) * self.single_transition_residual_gain
        scale = self.branch_scaler
        zero = pair.new_zeros(())
        b_tri_out = _gain(s) * scale(self.tri_mul_out(pair, pair_mask))
        pair = ops.dropout_add(pair, b_tri_out, p, tr, -3)
        b_tri_in = _gain(s) * scale(self.tri_mul_in(pair, pair_mask))
        pair = ops.dropout_add(pair, b_tri_in, p, tr, -3)
        if self.use_triangle_attention:
            b_row = _gain(s) * scale(self.pair_attn_row(pair, pair_mask))
            pair = ops.dropout_add(pair, b_row, p, tr, -3)
            b_col = _gain(s) * scale(self.pair_attn_col(pair, pair_mask))
            pair = ops.dropout_add(pair, b_col, p, tr, -2)
        else:
            b_row = b_col = zero
        b_pair_ffn = _gain(s_pf) * scale(map_pair_transition(self.pair_transition, pair, self.pair_chunk_budget, 4))
        pair = pair + b_pair_ffn
        if self.use_single_track:
            logits = self._single_bias(pair)
            b_single_attn = _gain(s) * scale(self.single_attn(single, seq_mask, logits))
            single = single + b_single_attn
            update = self.single_transition(single)
            probe = getattr(self, "_probe", None)
            if probe is not None and probe.enabled:
                probe.record_block(self._probe_layer_idx, single, update, s_sf)
            b_single_ffn = _gain(s_sf) * scale(update)
        else:
            b_single_attn = b_single_ffn = zero
        meter = getattr(self, "_act_meter", None)
        if meter is not None and getattr(meter, "enabled", False):
            meter.record_all_branches(
                self._act_layer_idx, b_tri_out=b_tri_out, b_tri_in=b_tri_in, b_pair_attn_row=b_row,
                b_pair_attn_col=b_col, b_pair_ffn=b_pair_ffn, b_single_attn=b_single_attn, b_single_ffn=b_single_ffn,
            )  # fmt: skip
        if self.use_single_track:
            single = single + b_single_ffn
        return pair, single


class Evoformer(nn.Module):
    """Embedders + MSA stack + Pairformer stack (reference: evoformer.py:358-608)."""

    def __init__(self, cfg, pf_cfg, template_cfg=None, optim=None):
        super().__init__()
        self._grad_checkpoint = bool(optim and optim.use_gradient_checkpointing)
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        c_msa, c_pair, c_single = cfg.msa_channel, cfg.pair_channel, cfg.seq_channel
        # raw token features (63) + conditioning-encoder output (seq_channel wide): 447 at the default width
        tf_dim = 63 + c_single
        self.template_embedding = TemplateEmbedding(template_cfg, optim=optim) if template_cfg is not None else None
        self.msa_activations = LinearNoBias(MSA_FEAT_DIM, c_msa)
        self.extra_msa_target_feat = LinearNoBias(tf_dim, c_msa)
        self.left_single = LinearNoBias(tf_dim, c_pair)
        self.right_single = LinearNoBias(tf_dim, c_pair)
        self.bond_embedding = LinearNoBias(1, c_pair)
        self.prev_embedding_layer_norm = LayerNorm(c_pair)
        self.prev_embedding = LinearNoBias(c_pair, c_pair, initializer="zeros")
        self.use_single_track = bool(pf_cfg.use_single_track)
        if self.use_single_track:
            self.prev_single_embedding_layer_norm = LayerNorm(c_single)
            self.prev_single_embedding = LinearNoBias(c_single, c_single, initializer="zeros")
        rel_dim = 2 * (2 * cfg.max_relative_idx + 2) + 1 + (2 * cfg.max_relative_chain + 2)
        self.position_activations = LinearNoBias(rel_dim, c_pair)
        self.single_activations = LinearNoBias(tf_dim, c_single)
        self.msa_stack = nn.ModuleList(
            EvoformerBlock(
                c_msa, c_pair, cfg.msa_attention.num_head, cfg.pair_attention.num_head, cfg.outer_product_num_channel,
                cfg.msa_dropout, cfg.pair_dropout, optim,
                block_residual_scale(i, cfg.num_layer, cfg.residual_output_scaling, cfg.uniform_residual_scale),
                cfg.use_triangle_attention, trimul_kwargs(cfg),
            )  # fmt: skip
            for i in range(cfg.num_layer)
        )
        self.trunk_pairformer = nn.ModuleList(
            PairFormerBlock(
                c_pair, c_single,
                num_pair_heads=pf_cfg.pair_attention.num_head,
                num_single_heads=pf_cfg.single_attention_num_head,
                single_key_dim=pf_cfg.single_key_dim,
                single_value_dim=pf_cfg.single_value_dim,
                pair_dropout=pf_cfg.pair_dropout,
                optim=optim,
                residual_out_scale=block_residual_scale(
                    i, pf_cfg.num_layer, pf_cfg.residual_output_scaling, pf_cfg.uniform_residual_scale
                ),
                pair_bias_gate=pf_cfg.pair_bias_gate,
                pair_bias_gate_init_tau=pf_cfg.pair_bias_gate_init_tau,
                single_transition_linear_out_init_gain=pf_cfg.single_transition_linear_out_init_gain,
                single_transition_residual_gain=resolve_branch_residual_gain(
                    i, pf_cfg.single_transition_residual_gain, pf_cfg.single_transition_residual_per_layer_extra
                ),
                pair_transition_residual_gain=resolve_branch_residual_gain(
                    i, pf_cfg.pair_transition_residual_gain, pf_cfg.pair_transition_residual_per_layer_extra
                ),
                branch_scaler=pf_cfg.branch_scaler,
                use_triangle_attention=pf_cfg.use_triangle_attention,
                use_single_track=pf_cfg.use_single_track,
                trimul_kwargs=trimul_kwargs(pf_cfg),
            )  # fmt: skip
            for i in range(pf_cfg.num_layer)
        )

    def forward(self, target_feat, msa_feat, rel_feat, pair_mask, seq_mask, msa_mask, prev_pair, prev_single,
                bond_matrix=None, template_aatype=None, template_pseudo_beta=None, template_pseudo_beta_mask=None,
                template_backbone_frame=None, template_backbone_mask=None, multichain_mask=None, template_ca=None,
                template_mask=None):  # fmt: skip
        pair = self.left_single(target_feat).unsqueeze(-2) + self.right_single(target_feat).unsqueeze(-3)
        pair = pair + map_pair_rows(
            lambda rows: self.prev_embedding(self.prev_embedding_layer_norm(rows)), prev_pair, self.pair_chunk_budget,
            4 * prev_pair.shape[-1],
        )  # fmt: skip
        pair = pair + self.position_activations(rel_feat)
        if bond_matrix is not None:
            pair = pair + self.bond_embedding(bond_matrix)
        if self.template_embedding is not None and template_aatype is not None:
            t_axis = 1 if template_aatype.dim() == 3 else 0
            if template_aatype.shape[t_axis] > 0:
                if multichain_mask is None:
                    multichain_mask = pair.new_ones(pair.shape[:-1])
                pair = pair + self.template_embedding(
                    query_pair=pair, template_aatype=template_aatype, template_pseudo_beta=template_pseudo_beta,
                    template_pseudo_beta_mask=template_pseudo_beta_mask,
                    template_backbone_frame=template_backbone_frame, template_backbone_mask=template_backbone_mask,
                    pair_mask=pair_mask, multichain_mask=multichain_mask, template_ca=template_ca,
                    template_mask=template_mask,
                )  # fmt: skip
        single = self.single_activations(target_feat)
        if self.use_single_track:
            single = single + self.prev_single_embedding(self.prev_single_embedding_layer_norm(prev_single))
        msa = self.msa_activations(msa_feat) + self.extra_msa_target_feat(target_feat).unsqueeze(-3)

        comm = getattr(self, "_axial_comm", None)
        if comm is not None and comm.world > 1 and not torch.is_grad_enabled() and pair.shape[-2] % comm.world == 0:
            # inference on several GPUs: both stacks run on row shards of the pair tensor
            from ..parallel.axial import sharded_trunk

            b1 = (lambda t: t[None]) if pair.dim() == 3 else (lambda t: t)
            msa, pair, single = sharded_trunk(self.msa_stack, self.trunk_pairformer, b1(msa), b1(pair), b1(single),
                                              b1(msa_mask), b1(pair_mask), b1(seq_mask), comm)  # fmt: skip
            if pair_mask.dim() == 2:
                msa, pair, single = msa[0], pair[0], single[0]
            return {"pair": pair, "single": single, "msa": msa, "target_feat": target_feat}
        use_ckpt = self._grad_checkpoint and torch.is_grad_enabled()
        for layer in self.msa_stack:
            if use_ckpt:
                msa, pair = _ckpt(layer, msa, pair, msa_mask, pair_mask)
            else:
                msa, pair = layer(msa, pair, msa_mask, pair_mask)
        meter = getattr(self, "_act_meter", None)
        if meter is not None:
            meter.record(0, single, pair)
        for i, layer in enumerate(self.trunk_pairformer):
            single_in, pair_in = single, pair
            if use_ckpt:
                pair, single = _ckpt(layer, pair, single, pair_mask, seq_mask)
            else:
                pair, single = layer(pair, single, pair_mask, seq_mask)
            if meter is not None:
                meter.record(i + 1, single, pair)
                meter.record_branch(i, single - single_in, pair - pair_in)
        return {"pair": pair, "single": single, "msa": msa, "target_feat": target_feat}
