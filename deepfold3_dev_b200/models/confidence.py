"""Confidence head: 4 Pairformer blocks per sample → pLDDT, PAE, PDE, experimentally-resolved logits.

Reference: model/confidence.py:38-337.
"""

from __future__ import annotations

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .embedders import DGRAM_NUM_BINS, dgram_from_positions
from .evoformer import PairFormerBlock, resolve_branch_residual_gain
from .precision import fp32_scope
from .primitives import LayerNorm, LinearNoBias, block_residual_scale, budget_rows, map_row_chunks


def _ckpt(fn, *args):
    return checkpoint(fn, *args, use_reentrant=False, determinism_check="none")


class ConfidenceHead(nn.Module):
    def __init__(self, cfg, target_feat_dim: int = 447, optim=None, fp32: bool = False):
        super().__init__()
        c_pair, c_single = cfg.pair_channel, cfg.seq_channel
        self.fp32 = fp32
        self._grad_checkpoint = bool(optim and optim.use_gradient_checkpointing)
        self.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.left_target_feat_project = LinearNoBias(target_feat_dim, c_pair)
        self.right_target_feat_project = LinearNoBias(target_feat_dim, c_pair)
        self.distogram_feat_project = LinearNoBias(DGRAM_NUM_BINS, c_pair)
        self.layers = nn.ModuleList(
            PairFormerBlock(
                c_pair=c_pair, c_single=c_single, num_pair_heads=cfg.pair_attention_num_head,
                num_single_heads=cfg.single_attention_num_head, single_key_dim=c_single, single_value_dim=c_single,
                optim=optim,
                residual_out_scale=block_residual_scale(
                    i, cfg.num_layer, cfg.residual_output_scaling, cfg.uniform_residual_scale
                ),
                pair_bias_gate=cfg.pair_bias_gate, pair_bias_gate_init_tau=cfg.pair_bias_gate_init_tau,
                single_transition_linear_out_init_gain=cfg.single_transition_linear_out_init_gain,
                single_transition_residual_gain=resolve_branch_residual_gain(
                    i, cfg.single_transition_residual_gain, cfg.single_transition_residual_per_layer_extra
                ),
                pair_transition_residual_gain=resolve_branch_residual_gain(
                    i, cfg.pair_transition_residual_gain, cfg.pair_transition_residual_per_layer_extra
                ),
                branch_scaler=cfg.branch_scaler,
            )  # fmt: skip
            for i in range(cfg.num_layer)
        )
        atoms = cfg.max_atoms_per_token
        self.plddt_logits_ln = LayerNorm(c_single)
        self.plddt_logits = LinearNoBias(c_single, atoms * cfg.num_plddt_bins, initializer="zeros")
        self.pae_logits_ln = LayerNorm(c_pair)
        self.pae_logits = LinearNoBias(c_pair, cfg.num_distogram_bins, initializer="zeros")
        self.pde_logits_ln = LayerNorm(c_pair)
        self.pde_half_logits = LinearNoBias(c_pair, cfg.num_distogram_bins, initializer="zeros")
        self.exp_resolved_ln = LayerNorm(c_single)
        self.exp_resolved_logits = LinearNoBias(c_single, atoms * 2, initializer="zeros")

    def _embed_features(self, target_feat, positions, pair_mask):
        out = self.left_target_feat_project(target_feat).unsqueeze(-2)
        out = out + self.right_target_feat_project(target_feat).unsqueeze(-3)
        with fp32_scope(self.fp32, positions.device.type):
            dgram = dgram_from_positions(positions.float() if self.fp32 else positions) * pair_mask[..., None]
        return out + self.distogram_feat_project(dgram.to(out.dtype))

    def _one_sample(self, pair, single, target_feat, positions, pair_mask, seq_mask, return_pre_logits):
        pair_act = pair + self._embed_features(target_feat, positions, pair_mask)
        single_act = single
        use_ckpt = self._grad_checkpoint and torch.is_grad_enabled()
        for layer in self.layers:
            if use_ckpt:
                pair_act, single_act = _ckpt(layer, pair_act, single_act, pair_mask, seq_mask)
            else:
                pair_act, single_act = layer(pair_act, single_act, pair_mask, seq_mask)
        rows = 0
        if not return_pre_logits and not torch.is_grad_enabled():
            rows = budget_rows(self.pair_chunk_budget, pair_act.shape[-2], 4 * pair_act.shape[-1])
        with fp32_scope(self.fp32, pair.device.type):
            cast = (lambda t: t.float()) if self.fp32 else (lambda t: t)
            s = cast(single_act)
            plddt = self.plddt_logits(self.plddt_logits_ln(s))
            resolved = self.exp_resolved_logits(self.exp_resolved_ln(s))
            if rows:
                pae = map_row_chunks(lambda r: self.pae_logits(self.pae_logits_ln(cast(r))), pair_act, rows)
                half = map_row_chunks(lambda r: self.pde_half_logits(self.pde_logits_ln(cast(r))), pair_act, rows)
                return plddt, resolved, pae, half + half.transpose(-3, -2)
            z = cast(pair_act)
            if return_pre_logits:
                return plddt, resolved, self.pae_logits_ln(z), self.pde_logits_ln(z)
            half = self.pde_half_logits(self.pde_logits_ln(z))
            return plddt, resolved, self.pae_logits(self.pae_logits_ln(z)), half + half.transpose(-3, -2)

    def forward(self, pair, single, pair_mask, seq_mask, target_feat, atom_positions, rep_atom_index=None,
                return_pre_logits: bool = False):  # fmt: skip
        """``atom_positions`` ``[B?, S, N, M, 3]``; outputs stacked on the sample axis (dim 0, or 1 when batched)."""
        batched = pair.dim() == 4
        N, dev = pair.shape[-3], pair.device
        axis = 1 if batched else 0
        S = atom_positions.shape[axis]
        if rep_atom_index is None:
            rep_atom_index = torch.ones(pair.shape[:-3] + (N,), dtype=torch.long, device=dev)
        idx = rep_atom_index.reshape(*rep_atom_index.shape, 1, 1).expand(*rep_atom_index.shape, 1, 3)
        prealloc = not torch.is_grad_enabled()
        outs: list = [[], [], [], []]
        for s in range(S):
            pos_s = atom_positions.select(axis, s)  # [B?, N, M, 3]
            positions = torch.gather(pos_s, -2, idx).squeeze(-2)  # [B?, N, 3]
            args = (pair, single, target_feat, positions, pair_mask, seq_mask, return_pre_logits)
            res = _ckpt(self._one_sample, *args) if torch.is_grad_enabled() else self._one_sample(*args)
            for k, x in enumerate(res):
                if not prealloc:
                    outs[k].append(x)
                    continue
                if s == 0:
                    shape = list(x.shape)
                    shape.insert(axis, S)
                    outs[k] = x.new_empty(shape)
                outs[k].select(axis, s).copy_(x)
            del res
        if not prealloc:
            outs = [torch.stack(xs, dim=axis) for xs in outs]
        plddt, resolved, pae, pde = outs
        out = {"plddt_logits": plddt, "exp_resolved_logits": resolved}
        if return_pre_logits:
            out["pae_features"], out["pde_features"] = pae, pde
        else:
            out["pae_logits"], out["pde_logits"] = pae, pde
        return out
