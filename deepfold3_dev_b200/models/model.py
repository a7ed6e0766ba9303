"""Top-level model: conditioning encoder → trunk with recycling → diffusion head → confidence and distogram heads.

Public surface equals the reference's (model/model.py:50-1187): ``DeepFold3(cfg)``,
``forward``, ``forward_training``, ``run_evoformer``, ``sample_from_trunk``,
``compute_distogram`` and a ``state_dict`` with the same keys.
"""

from __future__ import annotations

import dataclasses
from collections.abc import Sequence
import os
from contextlib import nullcontext

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from ..config.schema import DistogramConfig, ModelConfig, OptimConfig
from ..utils.cuda_graph import GraphCache, TrainGraphCache
from .atom_attention import EvoformerConditioningEncoder
from .confidence import ConfidenceHead
from .diffusion import DiffusionHead, GuidanceTerm
from .embedders import compute_rel_feat_dim, create_relative_encoding
from .evoformer import Evoformer
from .masked_msa import MaskedMSAHead, apply_bert_mask
from .precision import fp32_scope
from .primitives import LayerNorm, LinearNoBias, map_pair_rows, small_normal_init_

RAW_TARGET_FEAT_DIM = 63  # one-hot residue type (31) + profile (31) + deletion mean (1)
AATYPE_NUM_CLASSES = 31
MSA_NUM_CLASSES = 32


@dataclasses.dataclass
class DeepFold3Output:
    atom_positions: torch.Tensor  # [S, N, M, 3]
    atom_mask: torch.Tensor  # [S, N, M]
    plddt: torch.Tensor | None  # [S, N, M * bins]
    pae: torch.Tensor | None  # [S, N, N, 64]
    pde: torch.Tensor | None  # [S, N, N, 64]
    exp_resolved: torch.Tensor | None  # [S, N, M * 2]
    distogram: torch.Tensor | None  # [N, N, 64]


class DistogramHead(nn.Module):
    """``half_logits(pair)`` symmetrised over (i, j) (reference: model.py:60-131)."""

    def __init__(self, pair_channels=128, cfg: DistogramConfig | None = None, fp32=False, use_half_logits_ln=None):
        super().__init__()
        cfg = cfg or DistogramConfig()
        self.num_bins, self.first_break, self.last_break = cfg.num_bins, cfg.first_break, cfg.last_break
        self.fp32 = fp32
        if use_half_logits_ln is None:
            use_half_logits_ln = bool(getattr(cfg, "use_half_logits_ln", False))
        self.half_logits_ln = LayerNorm(pair_channels) if use_half_logits_ln else None
        self.half_logits = LinearNoBias(pair_channels, self.num_bins)
        self.pair_chunk_budget = 0
        alpha = float(getattr(cfg, "half_logits_init_alpha", 0.0))
        if alpha == 0.0:
            nn.init.zeros_(self.half_logits.weight)
        else:
            small_normal_init_(self.half_logits.weight, alpha)

    def _half(self, pair):
        z = pair.float() if self.fp32 else pair
        if self.half_logits_ln is not None:
            z = self.half_logits_ln(z)
        return self.half_logits(z)

    def forward(self, pair):
        with fp32_scope(self.fp32, pair.device.type):
            h = map_pair_rows(self._half, pair, self.pair_chunk_budget, 4 * pair.shape[-1])
        return h + h.transpose(-3, -2)

    def expected_distance(self, pair):
        probs = self.forward(pair).softmax(dim=-1)
        breaks = torch.linspace(self.first_break, self.last_break, self.num_bins - 1, device=pair.device)
        lower = torch.cat([breaks.new_zeros(1), breaks])
        upper = torch.cat([breaks, breaks[-1:] + (breaks[-1] - breaks[-2])])
        return (probs * (lower + upper) * 0.5).sum(-1)


class DeepFold3(nn.Module):
    def __init__(self, cfg: ModelConfig | None = None):
        super().__init__()
        cfg = cfg or ModelConfig()
        cfg.optim.require_backends()
        self.cfg = cfg
        ec, pfc, dc, cc = cfg.evoformer, cfg.pairformer, cfg.diffusion, cfg.confidence
        aca = dc.atom_cross_att
        self.evo_cond_encoder = EvoformerConditioningEncoder(
            per_atom_channels=aca.per_atom_channels, per_token_channels=ec.seq_channel,
            per_atom_pair_channels=aca.per_atom_pair_channels, num_blocks=aca.atom_transformer.num_blocks,
            Q=aca.queries_subset_size, K=aca.keys_subset_size, num_element_classes=aca.num_element_classes,
            num_atom_name_chars=aca.num_atom_name_chars, atom_name_length=aca.atom_name_length,
            ref_element_zero_index=aca.ref_element_zero_index,
        )  # fmt: skip
        self.evoformer = Evoformer(ec, pfc, template_cfg=cfg.template, optim=cfg.optim)
        rel_dim = compute_rel_feat_dim(ec.max_relative_idx, ec.max_relative_chain)
        self.diffusion_head = DiffusionHead(
            dc, c_single=ec.seq_channel, c_pair=ec.pair_channel, rel_feat_dim=rel_dim, optim=cfg.optim,
            target_feat_dim=RAW_TARGET_FEAT_DIM + ec.seq_channel,
        )
        self.confidence_head = ConfidenceHead(
            cc, target_feat_dim=RAW_TARGET_FEAT_DIM + ec.seq_channel, optim=cfg.optim,
            fp32=cfg.precision.fp32_confidence_head,
        )
        self.distogram_head = DistogramHead(ec.pair_channel, cfg=cfg.distogram, fp32=cfg.precision.fp32_distogram_head)
        self.distogram_head.pair_chunk_budget = cfg.optim.pair_chunk_budget_bytes
        self.masked_msa_head = (
            MaskedMSAHead(cfg.masked_msa, c_msa=ec.msa_channel, c_single=ec.seq_channel)
            if cfg.masked_msa.enabled
            else None
        )

    def load_state_dict(self, state_dict, strict=True, assign=False):
        """Keys of fused-kernel wrappers that older checkpoints carry are dropped before loading."""
        markers = OptimConfig.FUSED_STATE_DICT_MARKERS
        kept = {k: v for k, v in state_dict.items() if not any(m in k for m in markers)}
        return super().load_state_dict(kept, strict=strict, assign=assign)

    # ------------------------------------------------------------------ features
    def _build_raw_target_feat(self, features):
        onehot = F.one_hot(features["res_type"], AATYPE_NUM_CLASSES).float()
        parts = [onehot]
        if "profile" in features:
            prof = features["profile"].float()
            if prof.shape[-1] < AATYPE_NUM_CLASSES:
                prof = F.pad(prof, (0, AATYPE_NUM_CLASSES - prof.shape[-1]))
            parts.append(prof[..., :AATYPE_NUM_CLASSES])
        else:
            parts.append(onehot)
        if "deletion_mean" in features:
            parts.append(features["deletion_mean"].float().unsqueeze(-1))
        else:
            parts.append(onehot.new_zeros(*onehot.shape[:-1], 1))
        return torch.cat(parts, dim=-1)

    def _build_msa_feat_from_tensors(self, msa, deletion_matrix=None):
        onehot = F.one_hot(msa, MSA_NUM_CLASSES).float()
        if deletion_matrix is None:
            return torch.cat([onehot, onehot.new_zeros(*msa.shape, 2)], dim=-1)
        d = deletion_matrix.float()
        return torch.cat(
            [onehot, d.clamp(0.0, 1.0).unsqueeze(-1), (torch.arctan(d / 3.0) * (2.0 / torch.pi)).unsqueeze(-1)],
            dim=-1,
        )

    def _build_msa_feat(self, features):
        return self._build_msa_feat_from_tensors(features["msa"], features.get("deletion_matrix"))

    @staticmethod
    def _ref_kwargs(features):
        return {
            "ref_pos": features["ref_pos"],
            "ref_mask": features["ref_mask"].float(),
            "ref_element": features["ref_element"],
            "ref_charge": features["ref_charge"].float(),
            "ref_atom_name_chars": features["ref_atom_name_chars"],
            "ref_space_uid": features.get("ref_space_uid"),
        }

    # ------------------------------------------------------------------ trunk
    def _select_msa(self, features, recycle_idx, num_recycles, rng, msa_precropped, crop_offset):
        """This recycle's ``(msa, mask, deletions)``: a pre-built crop, or a fresh random subsample
        of ``msa_crop_size`` rows (query row kept) plus, in training, the random-k row mask
        (reference: model.py:385-431)."""
        full_msa, full_mask = features["msa"], features["msa_mask"]
        full_del = features.get("deletion_matrix")
        dev = full_msa.device
        rows_dim = full_msa.dim() - 2
        S_full, crop = full_msa.shape[-2], self.cfg.msa_crop_size
        if msa_precropped:
            base = (crop_offset + recycle_idx) * crop
            return (
                full_msa.narrow(rows_dim, base, crop),
                full_mask.narrow(rows_dim, base, crop),
                full_del.narrow(rows_dim, base, crop) if full_del is not None else None,
            )
        msa, mask, dele = full_msa, full_mask, full_del
        if S_full > crop:
            perm = torch.randperm(S_full - 1, generator=rng) + 1
            idx = torch.cat([torch.zeros(1, dtype=torch.long), perm[: crop - 1]]).sort().values.to(dev)
            msa, mask = full_msa.index_select(rows_dim, idx), full_mask.index_select(rows_dim, idx)
            dele = full_del.index_select(rows_dim, idx) if full_del is not None else None
        if self.training:
            pool = msa.shape[rows_dim]
            k = int(torch.randint(1, S_full + 1, (1,), generator=rng).item())
            if k < pool:
                keep = torch.cat([torch.zeros(1, dtype=torch.long), (torch.randperm(pool - 1, generator=rng) + 1)[: k - 1]])
                active = torch.zeros(pool, dtype=mask.dtype, device=dev)
                active[keep.to(dev)] = 1
                shape = [1] * mask.dim()
                shape[rows_dim] = pool
                mask = mask * active.view(*shape)
        return msa, mask, dele

    def _graph_trunk(self, dev) -> bool:
        if dev.type != "cuda" or torch.is_grad_enabled() or os.environ.get("DF3_GRAPH_TRUNK", "1") == "0":
            return False
        meter = getattr(self.evoformer, "_act_meter", None)
        return not (meter is not None and getattr(meter, "enabled", False))

    def _graph_trunk_training(self, dev) -> bool:
        """Graph the gradient-carrying trunk pass: a CUDA device, bf16 kernels (autocast), every activation kept (no
        checkpointing, whose recomputation re-enters Python), no activation meter, and not switched off."""
        if dev.type != "cuda" or not torch.is_grad_enabled() or os.environ.get("DF3_GRAPH_TRAIN", "1") == "0":
            return False
        if self.cfg.optim.use_gradient_checkpointing or not torch.is_autocast_enabled("cuda"):
            return False
        meter = getattr(self.evoformer, "_act_meter", None)
        return not (meter is not None and getattr(meter, "enabled", False))

    def run_evoformer(self, features, num_recycles, seed=0, msa_precropped=False, crop_offset=0, mask_msa=False):
        """Feature building + ``num_recycles + 1`` trunk passes.

        Returns ``(embeddings, rel_feat, target_feat, seq_mask, pair_mask)``;
        works on unbatched ``[N, ...]`` and batched ``[B, N, ...]`` features.
        """
        dev = features["res_type"].device
        batched = features["res_type"].dim() >= 2
        N = features["res_type"].shape[-1]
        token_index = features.get("token_index")
        if token_index is None:
            token_index = torch.arange(N, dtype=torch.long, device=dev).expand_as(features["residue_index"])
        sym_id = features.get("sym_id")
        if sym_id is None:
            sym_id = torch.zeros_like(features["residue_index"])
        rel_feat = create_relative_encoding(
            token_index, features["residue_index"], features["asym_id"], features["entity_id"], sym_id,
            self.cfg.evoformer.max_relative_idx, self.cfg.evoformer.max_relative_chain,
        )  # fmt: skip
        raw_feat = self._build_raw_target_feat(features)

        ref = self._ref_kwargs(features)
        fp32_enc = self.cfg.precision.fp32_evo_cond_encoder
        # an fp32 island: autocast switched off, inputs are fp32 already
        ctx = torch.amp.autocast(device_type=dev.type, enabled=False) if fp32_enc else nullcontext()
        with ctx:
            args = (ref["ref_pos"], ref["ref_mask"], ref["ref_element"], ref["ref_charge"],
                    ref["ref_atom_name_chars"], ref["ref_space_uid"])  # fmt: skip
            if torch.is_grad_enabled() and self.cfg.optim.use_gradient_checkpointing:
                cond = checkpoint(self.evo_cond_encoder, *args, use_reentrant=False, determinism_check="none")
            else:
                cond = self.evo_cond_encoder(*args)
        target_feat = torch.cat([raw_feat, cond.to(raw_feat.dtype)], dim=-1)

        seq_mask, pair_mask = features["seq_mask"].float(), features["pair_mask"].float()
        c_pair, c_single = self.cfg.evoformer.pair_channel, self.cfg.evoformer.seq_channel
        if "_prev_pair" in features:
            prev_pair, prev_single = features["_prev_pair"], features["_prev_single"]
        else:
            lead = features["res_type"].shape[:-1]
            prev_pair = torch.zeros(*lead, N, N, c_pair, device=dev, dtype=target_feat.dtype)
            prev_single = torch.zeros(*lead, N, c_single, device=dev, dtype=target_feat.dtype)

        tmpl = {}
        if "template_aatype" in features:
            tmpl["template_aatype"] = features["template_aatype"]
            for key in ("template_pseudo_beta", "template_pseudo_beta_mask", "template_backbone_frame",
                        "template_backbone_mask"):  # fmt: skip
                tmpl[key] = features[key].float()
            for key in ("template_ca", "template_mask"):
                if key in features:
                    tmpl[key] = features[key].float()
        bond_matrix = features.get("bond_matrix")
        if bond_matrix is not None:
            bond_matrix = bond_matrix.to(dev).float()
        asym = features["asym_id"].to(dev)
        multichain_mask = (asym.unsqueeze(-1) == asym.unsqueeze(-2)).float()

        S_full, crop = features["msa"].shape[-2], self.cfg.msa_crop_size
        if msa_precropped and S_full < (crop_offset + num_recycles + 1) * crop:
            raise ValueError(
                f"msa_precropped: MSA pool {S_full} < required {(crop_offset + num_recycles + 1) * crop} "
                f"(crop={crop}, crop_offset={crop_offset}, num_recycles={num_recycles}). "
                "Featurizer msa_crop_size / n_msa_crops must match the model."
            )
        rng = torch.Generator(device="cpu").manual_seed(seed)
        bert = None
        embeddings = None
        for r in range(num_recycles + 1):
            msa, msa_mask, dele = self._select_msa(features, r, num_recycles, rng, msa_precropped, crop_offset)
            if mask_msa and self.masked_msa_head is not None:
                gen = torch.Generator(device=dev).manual_seed(int(seed) + r + 0x5EED)
                msa, true_msa, hit = apply_bert_mask(msa, msa_mask, features.get("profile"), self.cfg.masked_msa, gen)
                bert = (true_msa, hit, msa_mask)
            trunk_in = dict(
                target_feat=target_feat, msa_feat=self._build_msa_feat_from_tensors(msa, dele), rel_feat=rel_feat,
                pair_mask=pair_mask, seq_mask=seq_mask, msa_mask=msa_mask.float(), prev_pair=prev_pair,
                prev_single=prev_single, bond_matrix=bond_matrix, multichain_mask=multichain_mask, **tmpl,
            )  # fmt: skip
            if self._graph_trunk(dev):
                # no autograd on this pass: replay the whole trunk from a CUDA graph (captured once per shape)
                graphs = self.__dict__.setdefault("_trunk_graphs", GraphCache(max_graphs=4))
                embeddings = graphs.run(self.evoformer, trunk_in, mode=self.evoformer.training)
            elif self._graph_trunk_training(dev):
                # the pass that carries gradients: forward and backward each replay one captured graph
                graphs = self.__dict__.setdefault("_trunk_train_graphs", TrainGraphCache(max_graphs=1))
                embeddings = graphs.run(self.evoformer, trunk_in, self.evoformer.parameters(), mode=self.evoformer.training)
            else:
                embeddings = self.evoformer(**trunk_in)
            if r < num_recycles:
                prev_pair, prev_single = embeddings["pair"].detach(), embeddings["single"].detach()
        if bert is not None:
            embeddings["true_msa"], embeddings["bert_mask"], embeddings["bert_msa_valid_mask"] = bert
        return embeddings, rel_feat, target_feat, seq_mask, pair_mask

    # ------------------------------------------------------------------ training
    def forward_training(self, features, num_recycles, diffusion_batch_size, mini_rollout_steps=20,
                         mini_rollout_samples=1, seed=0, fused_ce=False, diffusion_chunk_size=0, backward_fn=None,
                         loss_cfg=None, compute_confidence=True, msa_precropped=False, chain_perm_gate_k=1,
                         permute_gt_before_noise=False, compute_diffusion=True):  # fmt: skip
        """Training forward (reference: model.py:493-959).

        1. trunk: ``num_recycles`` passes without grad, then one with grad;
        2. mini-rollout without grad (feeds chain/atom symmetry resolution and the confidence head);
        3. diffusion training on ``diffusion_batch_size`` noise samples, optionally in chunks whose
           loss is back-propagated through ``backward_fn`` as soon as it is computed;
        4. confidence head on detached trunk outputs; 5. distogram head.
        """
        from ..training import objective as L
        from ..training.collectives import slice_batch_dict

        ref = self._ref_kwargs(features)
        if num_recycles > 0:
            with torch.no_grad():
                warm = self.run_evoformer(features, num_recycles - 1, seed=seed, msa_precropped=msa_precropped)[0]
            features["_prev_pair"], features["_prev_single"] = warm["pair"], warm["single"]
        do_mask = self.masked_msa_head is not None and self.training
        embeddings, rel_feat, target_feat, seq_mask, pair_mask = self.run_evoformer(
            features, 0, seed=seed + num_recycles, msa_precropped=msa_precropped, crop_offset=num_recycles,
            mask_msa=do_mask,
        )  # fmt: skip
        features.pop("_prev_pair", None)
        features.pop("_prev_single", None)
        embeddings["target_feat"] = target_feat
        pred: dict = {"single": embeddings["single"], "pair": embeddings["pair"]}

        if self.masked_msa_head is not None and "bert_mask" in embeddings:
            args = (embeddings["msa"], embeddings["single"], embeddings["bert_msa_valid_mask"])
            if torch.is_grad_enabled() and self.cfg.optim.use_gradient_checkpointing:
                logits = checkpoint(self.masked_msa_head, *args, use_reentrant=False, determinism_check="none")
            else:
                logits = self.masked_msa_head(*args)
            pred["masked_msa_logits"] = logits
            pred["true_msa"], pred["bert_mask"] = embeddings["true_msa"], embeddings["bert_mask"]

        # 2. mini-rollout
        head = self.diffusion_head
        dcfg = head.cfg
        with torch.no_grad():
            keep = (dcfg.steps, dcfg.num_samples)
            dcfg.steps, dcfg.num_samples = mini_rollout_steps, max(mini_rollout_samples, chain_perm_gate_k)
            was_training = head.training
            head.eval()
            try:
                mini = head.sample(
                    embeddings={k: v.detach() for k, v in embeddings.items()}, seq_mask=seq_mask,
                    rel_feat=rel_feat.detach(), guidance=False,
                    **{k: (v.detach() if isinstance(v, torch.Tensor) else v) for k, v in ref.items()},
                )  # fmt: skip
            finally:
                dcfg.steps, dcfg.num_samples = keep
                head.train(was_training)
        mini_full = mini["atom_positions"].detach()
        if chain_perm_gate_k > 1:
            pred["chain_perm_gate_pos"] = mini_full
            pred["mini_rollout_pos"] = mini_full[:, :mini_rollout_samples]
        else:
            pred["mini_rollout_pos"] = mini_full

        # 2b. permute the ground truth once, before noise is added to it
        gt_pos, gt_mask = features["atom_gt_positions"], features["atom_gt_mask"]
        if permute_gt_before_noise and pred.get("mini_rollout_pos") is not None:
            B_gt, N_tok = gt_pos.shape[0], gt_pos.shape[1]
            new_pos, new_mask = torch.empty_like(gt_pos), torch.empty_like(gt_mask)
            cp_index = torch.arange(N_tok, device=gt_pos.device).expand(B_gt, N_tok).contiguous()
            cp_keep = torch.ones(B_gt, N_tok, dtype=torch.bool, device=gt_pos.device)
            for b in range(B_gt):
                pred_b = {"mini_rollout_pos": pred["mini_rollout_pos"][b]}
                if "chain_perm_gate_pos" in pred:
                    pred_b["chain_perm_gate_pos"] = pred["chain_perm_gate_pos"][b]
                gp, gm, ci, ck = L.permute_gt_for_diffusion(
                    pred_b, slice_batch_dict(features, b, B_gt), stability_gate_k=chain_perm_gate_k
                )
                new_pos[b], new_mask[b] = gp, gm
                if ci is not None:
                    cp_index[b], cp_keep[b] = ci, ck
            gt_pos, gt_mask = new_pos, new_mask
            features["__gt_prepermuted__"] = True
            features["chain_perm_index"], features["chain_perm_keep"] = cp_index, cp_keep

        # 3. diffusion training
        if compute_diffusion:
            self._diffusion_training(
                pred, features, embeddings, target_feat, rel_feat, seq_mask, ref, gt_pos, gt_mask,
                diffusion_batch_size, diffusion_chunk_size, backward_fn, loss_cfg,
            )  # fmt: skip

        # 4. confidence head on detached inputs
        if compute_confidence:
            conf_pair = embeddings["pair"].detach()
            if self.training and self.cfg.confidence.use_pair_emb_prob < 1.0:
                if not bool(torch.rand(()) < self.cfg.confidence.use_pair_emb_prob):
                    conf_pair = conf_pair * 0
            conf = self.confidence_head(
                pair=conf_pair, single=embeddings["single"].detach(), pair_mask=pair_mask, seq_mask=seq_mask,
                target_feat=target_feat.detach(), atom_positions=pred["mini_rollout_pos"],
                rep_atom_index=features.get("token_to_rep_atom"), return_pre_logits=fused_ce,
            )  # fmt: skip
            pred["plddt"], pred["exp_resolved"] = conf["plddt_logits"], conf["exp_resolved_logits"]
            if fused_ce:
                pred["pae_features"], pred["pde_features"] = conf["pae_features"], conf["pde_features"]
                pred["pae_weight"] = self.confidence_head.pae_logits.weight
                pred["pde_weight"] = self.confidence_head.pde_half_logits.weight
            else:
                pred["pae"], pred["pde"] = conf["pae_logits"], conf["pde_logits"]

        # 5. distogram
        if fused_ce:
            pred["distogram_features"] = embeddings["pair"]
            pred["distogram_weight"] = self.distogram_head.half_logits.weight
        else:
            pred["distogram"] = self.distogram_head(embeddings["pair"])
        return pred

    def _diffusion_training(self, pred, features, embeddings, target_feat, rel_feat, seq_mask, ref, gt_pos, gt_mask,
                            diffusion_batch_size, diffusion_chunk_size, backward_fn, loss_cfg):  # fmt: skip
        from ..training import objective as L
        from .diffusion import (
            build_diffusion_clean_mask,
            cond_drop_stats,
            draw_interface_pair_keep,
            mask_trunk_pair,
            null_pair_stats,
        )

        head = self.diffusion_head
        dcfg = head.cfg
        use_cond = True
        if self.training and dcfg.use_conditioning_prob < 1.0:
            use_cond = bool(torch.rand(()) < dcfg.use_conditioning_prob)
        pair_keep = None
        if (not use_cond and dcfg.cond_drop_interface_frac > 0.0 and features.get("asym_id") is not None
                and bool(torch.rand(()) < dcfg.cond_drop_interface_frac)):  # fmt: skip
            pair_keep = draw_interface_pair_keep(features["asym_id"], seq_mask)
            if pair_keep is not None:
                use_cond = True
        if self.training and dcfg.use_conditioning_prob < 1.0:
            pred["__cond_drop__"] = cond_drop_stats(
                features.get("asym_id"), seq_mask, use_conditioning=use_cond, pair_keep=pair_keep
            )
        if self.training and head.null_pair is not None:
            pred["__null_pair__"] = null_pair_stats(head.null_pair, embeddings["pair"], features.get("asym_id"), seq_mask)
        clean_mask = None
        if self.training and dcfg.diffusion_mask_prob > 0.0 and features.get("asym_id") is not None:
            clean_mask = build_diffusion_clean_mask(
                features["asym_id"], seq_mask, diffusion_batch_size, prob=dcfg.diffusion_mask_prob,
                mode=dcfg.diffusion_mask_mode, min_frac=dcfg.diffusion_mask_min_frac,
                max_frac=dcfg.diffusion_mask_max_frac,
            )  # fmt: skip

        chunked = (diffusion_chunk_size > 0 and backward_fn is not None and loss_cfg is not None
                   and diffusion_batch_size % diffusion_chunk_size == 0)  # fmt: skip
        if not chunked:
            emb = embeddings if pair_keep is None else mask_trunk_pair(embeddings, pair_keep, head.null_pair)
            gt_aug, denoised, noise_levels = head.sample_training(
                gt_positions=gt_pos, gt_mask=gt_mask, embeddings=emb, seq_mask=seq_mask, rel_feat=rel_feat,
                num_samples=diffusion_batch_size, clean_mask=clean_mask, use_conditioning=use_cond, **ref,
            )  # fmt: skip
            pred["denoised"], pred["gt_augmented"], pred["noise_levels"] = denoised, gt_aug, noise_levels
            if clean_mask is not None:
                pred["diffusion_clean_mask"] = clean_mask
            return

        # chunked: trunk outputs become leaves; each chunk's loss is back-propagated at once and the
        # leaf gradients are pushed through the trunk in one walk afterwards
        real = (embeddings["pair"], embeddings["single"], target_feat)
        leaves = tuple(t.detach().requires_grad_(t.requires_grad) for t in real)
        emb_det = {"pair": leaves[0], "single": leaves[1], "target_feat": leaves[2]}
        chunks = diffusion_batch_size // diffusion_chunk_size
        B = real[0].shape[0]
        logged: dict = {}
        total = real[0].new_zeros(())
        mini_pos = pred["mini_rollout_pos"]
        for c in range(chunks):
            cm = None if clean_mask is None else clean_mask[:, c * diffusion_chunk_size : (c + 1) * diffusion_chunk_size]
            emb_c = emb_det if pair_keep is None else mask_trunk_pair(emb_det, pair_keep, head.null_pair)
            gt_aug, denoised, noise_levels = head.sample_training(
                gt_positions=gt_pos, gt_mask=gt_mask, embeddings=emb_c, seq_mask=seq_mask, rel_feat=rel_feat,
                num_samples=diffusion_chunk_size, clean_mask=cm, use_conditioning=use_cond, **ref,
            )  # fmt: skip
            chunk_loss = real[0].new_zeros(())
            comps: dict = {}
            for b in range(B):
                pred_b = {"denoised": denoised[b], "gt_augmented": gt_aug[b], "noise_levels": noise_levels[b],
                          "mini_rollout_pos": mini_pos[b]}  # fmt: skip
                if cm is not None:
                    pred_b["diffusion_clean_mask"] = cm[b]
                if "chain_perm_gate_pos" in pred:
                    pred_b["chain_perm_gate_pos"] = pred["chain_perm_gate_pos"][b]
                feats_b = {
                    k: (v[b] if isinstance(v, torch.Tensor) and v.dim() >= 1 and v.shape[0] == B else v)
                    for k, v in features.items()
                }
                loss_b, comp_b = L.diffusion_only_loss(pred_b, feats_b, loss_cfg)
                chunk_loss = chunk_loss + loss_b / B
                for k, v in comp_b.items():
                    comps[k] = comps.get(k, v.new_zeros(())) + v / B
            backward_fn(chunk_loss / chunks)
            total = total + chunk_loss.detach() / chunks
            for k, v in comps.items():
                logged[k] = logged.get(k, v.new_zeros(())) + v / chunks
        flow = [(t, d.grad) for t, d in zip(real, leaves) if d.grad is not None]
        if flow:
            torch.autograd.backward([t for t, _ in flow], [g for _, g in flow], retain_graph=True)
        pred["__diffusion_total__"], pred["__diffusion_logged__"] = total, logged

    # ------------------------------------------------------------------ inference
    def forward(self, features, seed=0, num_recycles=None, num_samples=None,
                guidance_terms: Sequence[GuidanceTerm] | None = None, restraints: Sequence = (),
                restraint_weight=0.0, restraint_rigid=True, restraint_max_step=2.0, restraint_after_step=False,
                restraint_after_sigma=16.0) -> DeepFold3Output:  # fmt: skip
        """Full prediction: trunk with recycling, ``num_samples`` diffusion samples, confidence, distogram."""
        if num_recycles is None:
            num_recycles = self.cfg.num_recycles
        trunk = self.run_evoformer(features, num_recycles, seed=seed)
        return self.sample_from_trunk(
            features, trunk, seed=seed, num_samples=num_samples, guidance_terms=guidance_terms,
            restraints=restraints, restraint_weight=restraint_weight, restraint_rigid=restraint_rigid,
            restraint_max_step=restraint_max_step, restraint_after_step=restraint_after_step,
            restraint_after_sigma=restraint_after_sigma,
        )  # fmt: skip

    def sample_from_trunk(self, features, trunk, seed=0, num_samples=None, guidance_terms=None, restraints=(),
                          restraint_weight=0.0, restraint_rigid=True, restraint_max_step=2.0,
                          restraint_after_step=False, restraint_after_sigma=16.0, distogram=None):  # fmt: skip
        """Everything after the trunk; several guidance settings can share one ``trunk`` (reference: :1029-1107)."""
        embeddings, rel_feat, target_feat, seq_mask, pair_mask = trunk
        dcfg = self.diffusion_head.cfg
        keep = dcfg.num_samples
        if num_samples is not None:
            dcfg.num_samples = num_samples
        try:
            dev = features["res_type"].device
            gen = torch.Generator(device=dev).manual_seed(seed)
            pair_keep = None
            if guidance_terms is None and dcfg.guidance_scale != 1.0 and dcfg.guidance_drop == "interface":
                from .diffusion import interface_pair_keep

                pair_keep = interface_pair_keep(features["asym_id"].to(dev))
            emb = dict(embeddings)
            emb.setdefault("target_feat", target_feat)
            sample = self.diffusion_head.sample(
                embeddings=emb, seq_mask=seq_mask, rel_feat=rel_feat, generator=gen, guidance_pair_keep=pair_keep,
                guidance_terms=guidance_terms, restraints=restraints, restraint_weight=restraint_weight,
                restraint_rigid=restraint_rigid, restraint_max_step=restraint_max_step,
                restraint_after_step=restraint_after_step, restraint_after_sigma=restraint_after_sigma,
                **self._ref_kwargs(features),
            )  # fmt: skip
            conf = self.confidence_head(
                pair=embeddings["pair"], single=embeddings["single"], pair_mask=pair_mask, seq_mask=seq_mask,
                target_feat=target_feat, atom_positions=sample["atom_positions"],
                rep_atom_index=features.get("token_to_rep_atom"),
            )  # fmt: skip
            disto = distogram if distogram is not None else self.distogram_head(embeddings["pair"])
            return DeepFold3Output(
                atom_positions=sample["atom_positions"], atom_mask=sample["mask"], plddt=conf["plddt_logits"],
                pae=conf["pae_logits"], pde=conf["pde_logits"], exp_resolved=conf["exp_resolved_logits"],
                distogram=disto,
            )  # fmt: skip
        finally:
            dcfg.num_samples = keep

    @torch.no_grad()
    def compute_distogram(self, features, num_recycles=None):
        """Trunk + distogram head only: ``[N, N, 64]`` logits."""
        if num_recycles is None:
            num_recycles = self.cfg.num_recycles
        return self.distogram_head(self.run_evoformer(features, num_recycles)[0]["pair"])
