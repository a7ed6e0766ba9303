"""Diffusion head: conditioning, atom encoder, 24-block transformer, atom decoder, sampler, training rollout.

Reference: model/diffusion.py:903-1775. One execution form serves training,
the mini-rollout and inference: per-molecule state is computed once
(``compute_static`` also hoists pair logits and atom-block terms) and every
denoiser call runs all samples of all molecules as ``[B, S, ...]``.
"""

from __future__ import annotations

import os
from collections.abc import Sequence
from contextlib import nullcontext

import torch
import torch.nn as nn
import torch.nn.functional as F
from torch.utils.checkpoint import checkpoint

from .. import ops
from . import denoise_graph
from .atom_attention import AtomDecoder, AtomEncoder
from .diffusion_modules import (  # noqa: F401 - re-exported API
    DiffusionConditioningBlock,
    DiffusionStatic,
    DiffusionTransformer,
    DiffusionTransformerBlock,
    GuidanceTerm,
    augment,
    build_diffusion_clean_mask,
    cond_drop_stats,
    draw_interface_pair_keep,
    interface_pair_keep,
    mask_trunk_pair,
    noise_schedule,
    null_pair_stats,
)
from .precision import upcast_fp32
from .primitives import LinearNoBias


def _batched(t, batched: bool):
    return t if (t is None or batched) else t.unsqueeze(0)


class DiffusionHead(nn.Module):
    def __init__(self, cfg, c_single=384, c_pair=128, rel_feat_dim=139, optim=None, target_feat_dim=447):
        super().__init__()
        self.cfg = cfg
        aca = cfg.atom_cross_att
        c_diff = aca.per_token_channels
        # recompute each denoiser call in backward (what the reference does) unless memory is plentiful:
        # DF3_DIFFUSION_CKPT=0 keeps the activations of all samples instead
        self._grad_checkpoint = os.environ.get("DF3_DIFFUSION_CKPT", "1") != "0"
        self.conditioning = DiffusionConditioningBlock(
            c_pair_in=c_pair, c_single_in=c_single, rel_feat_dim=rel_feat_dim,
            c_pair_out=cfg.conditioning_pair_channel, c_single_out=cfg.conditioning_seq_channel,
            target_feat_dim=target_feat_dim,
            use_trunk_single=cfg.conditioning_use_trunk_single, sigma_data=cfg.sigma_data,
            fourier_dim=cfg.fourier_dim, num_intermediate_factor=cfg.conditioning_num_intermediate_factor,
            optim=optim,
        )  # fmt: skip
        if cfg.cond_drop_fill == "learned":
            self.null_pair_dir = nn.Parameter(torch.zeros(c_pair))
            self.null_pair_log_scale = nn.Parameter(torch.zeros(()))
        self.atom_encoder = AtomEncoder(
            per_atom_channels=aca.per_atom_channels, per_token_channels=aca.per_token_channels,
            per_atom_pair_channels=aca.per_atom_pair_channels,
            atom_transformer_num_blocks=aca.atom_transformer.num_blocks, Q=aca.queries_subset_size,
            K=aca.keys_subset_size, num_element_classes=aca.num_element_classes,
            num_atom_name_chars=aca.num_atom_name_chars, atom_name_length=aca.atom_name_length,
            ref_element_zero_index=aca.ref_element_zero_index, c_trunk_single=c_single,
            c_trunk_pair=cfg.conditioning_pair_channel,
        )  # fmt: skip
        self.atom_encoder.pair_chunk_budget = optim.pair_chunk_budget_bytes if optim is not None else 0
        self.single_cond_emb_norm_w = nn.Parameter(torch.ones(cfg.conditioning_seq_channel))
        self.single_cond_embedding_projection = LinearNoBias(cfg.conditioning_seq_channel, c_diff, initializer="zeros")
        tc = cfg.transformer
        self.transformer = DiffusionTransformer(
            c=c_diff, c_single_cond=cfg.conditioning_seq_channel, num_blocks=tc.num_blocks, num_heads=tc.num_head,
            key_dim=tc.key_dim, value_dim=tc.value_dim, num_intermediate_factor=tc.num_intermediate_factor,
            super_block_size=tc.super_block_size, c_pair=cfg.conditioning_pair_channel, optim=optim,
            cond_bias_init_beta=tc.cond_bias_init_beta,
        )  # fmt: skip
        self.atom_decoder = AtomDecoder(
            per_atom_channels=aca.per_atom_channels, per_token_channels=c_diff,
            per_atom_pair_channels=aca.per_atom_pair_channels,
            atom_transformer_num_blocks=aca.atom_transformer.num_blocks,
        )  # fmt: skip

    # ---- learned fill of dropped pair conditioning ----
    @property
    def null_pair(self):
        if not hasattr(self, "null_pair_dir"):
            return None
        return self.null_pair_log_scale.exp() * self.null_pair_dir

    @torch.no_grad()
    def init_null_pair(self, vec: torch.Tensor) -> None:
        if not hasattr(self, "null_pair_dir"):
            raise ValueError("init_null_pair needs cond_drop_fill: learned")
        vec = vec.detach().float().to(self.null_pair_dir.device)
        if vec.shape != self.null_pair_dir.shape:
            raise ValueError(f"null_pair init has shape {tuple(vec.shape)}, expected {tuple(self.null_pair_dir.shape)}")
        rms = vec.pow(2).mean().sqrt()
        if rms > 0:
            self.null_pair_log_scale.fill_(rms.log())
            self.null_pair_dir.copy_(vec / rms)
        else:
            self.null_pair_log_scale.zero_()
            self.null_pair_dir.zero_()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        old = state_dict.pop(prefix + "null_pair", None)  # single-vector form of older checkpoints
        if old is not None and hasattr(self, "null_pair_dir"):
            rms = old.float().pow(2).mean().sqrt()
            scale = rms if rms > 0 else torch.ones(())
            state_dict[prefix + "null_pair_dir"] = (old.float() / scale).to(old.dtype)
            state_dict[prefix + "null_pair_log_scale"] = scale.log() if rms > 0 else torch.zeros(())
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    # ---- noise-independent state ----
    def compute_static(self, embeddings, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, seq_mask,
                       rel_feat, ref_space_uid=None, use_conditioning=True) -> DiffusionStatic:  # fmt: skip
        """Inputs ``[B, ...]``. With ``use_conditioning=False`` the trunk pair (and with
        ``cond_drop='both'`` the trunk single) is zeroed on its way into the conditioning block;
        the atom encoder still sees the real trunk single (reference: diffusion.py:1025-1084)."""
        cond_single, cond_pair = embeddings["single"], embeddings["pair"]
        if not use_conditioning:
            cond_pair = cond_pair * 0
            if self.null_pair is not None:
                cond_pair = cond_pair + self.null_pair.to(cond_pair.dtype)
            if self.cfg.cond_drop == "both":
                cond_single = cond_single * 0
        elif self.null_pair is not None and self.training and torch.is_grad_enabled():
            cond_single = cond_single + 0 * self.null_pair.sum().to(cond_single.dtype)
        pre_noise, pair_cond = self.conditioning.compute_static(
            cond_single, cond_pair, embeddings["target_feat"], rel_feat
        )
        enc_static = self.atom_encoder.compute_static(
            ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, embeddings["single"], pair_cond,
            ref_space_uid, decoder=self.atom_decoder,
        )  # fmt: skip
        logits = self.transformer.hoist_pair_logits(pair_cond, seq_mask)
        return DiffusionStatic(enc_static, pair_cond, pre_noise, ref_pos, ref_mask, seq_mask, logits)

    def hoist_static(self, static: DiffusionStatic, num_samples: int) -> DiffusionStatic:
        """API parity: the static built here is already in its hoisted, broadcast form."""
        return static

    # ---- one denoiser evaluation ----
    def _denoise_core(self, noisy_pos, noise_level, static: DiffusionStatic):
        """``noisy_pos`` ``[B, S, N, M, 3]``; ``noise_level`` ``[B, S]`` or ``[B, 1]`` (shared by the samples)."""
        sd = self.cfg.sigma_data
        m = static.ref_mask[:, None, :, :, None].to(noisy_pos.dtype)
        nl = noise_level.to(noisy_pos.dtype)[:, :, None, None, None]
        act_pos = noisy_pos * m / (nl**2 + sd**2).sqrt()
        single_cond = self.conditioning.add_noise(static.single_cond_pre_noise.unsqueeze(1), noise_level)
        enc = self.atom_encoder(act_pos, static.encoder_static)
        act = enc.token_act.float()
        sc = ops.layer_norm(single_cond, self.single_cond_emb_norm_w, None)
        act = act + self.single_cond_embedding_projection(sc)
        act = self.transformer.run(act, single_cond, static.pair_logits)
        update = self.atom_decoder(act, enc)
        skip = sd**2 / (nl**2 + sd**2)
        out_scale = nl * sd / (nl**2 + sd**2).sqrt()
        return (skip * noisy_pos + out_scale * update.to(noisy_pos.dtype)) * m

    def _denoise_samples(self, noisy_pos, noise_level, static: DiffusionStatic):
        if torch.is_grad_enabled() and self._grad_checkpoint:
            return checkpoint(self._denoise_core, noisy_pos, noise_level, static, use_reentrant=False,
                              determinism_check="none")  # fmt: skip
        return self._denoise_core(noisy_pos, noise_level, static)

    def denoise(self, noisy_pos, noise_level, embeddings=None, ref_pos=None, ref_mask=None, ref_element=None,
                ref_charge=None, ref_atom_name_chars=None, ref_space_uid=None, seq_mask=None, rel_feat=None,
                static=None, use_conditioning=True):  # fmt: skip
        """Reference-shaped single-sample call: ``noisy_pos`` ``[B?, N, M, 3]``, ``noise_level`` scalar or ``[B]``."""
        batched = noisy_pos.dim() == 4
        if static is None:
            static = self.compute_static(
                {k: _batched(v, batched) for k, v in embeddings.items()}, _batched(ref_pos, batched),
                _batched(ref_mask, batched), _batched(ref_element, batched), _batched(ref_charge, batched),
                _batched(ref_atom_name_chars, batched), _batched(seq_mask, batched), _batched(rel_feat, batched),
                _batched(ref_space_uid, batched), use_conditioning,
            )  # fmt: skip
        x = _batched(noisy_pos, batched).unsqueeze(1)
        nl = noise_level.reshape(-1, 1).expand(x.shape[0], 1) if noise_level.dim() <= 1 else noise_level
        out = self._denoise_core(x, nl, static).squeeze(1)
        return out if batched else out.squeeze(0)

    # ---- sampler ----
    @torch.no_grad()
    def sample(self, embeddings, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, seq_mask, rel_feat,
               generator=None, ref_space_uid=None, guidance=True, guidance_pair_keep=None, guidance_terms=None,
               restraints: Sequence = (), restraint_weight=0.0, restraint_rigid=True, restraint_max_step=2.0,
               restraint_after_step=False, restraint_after_sigma=16.0):  # fmt: skip
        """Euler sampler with stochastic churn (reference: diffusion.py:1325-1621).

        Unbatched inputs return ``atom_positions`` ``[S, N, M, 3]`` and ``mask``
        ``[S, N, M]``; batched inputs add a leading ``B``.
        """
        cfg = self.cfg
        terms: tuple[GuidanceTerm, ...] = ()
        if guidance and guidance_terms is not None:
            terms = tuple(t for t in guidance_terms if t.scale != 1.0)
        elif guidance and cfg.guidance_scale != 1.0:
            if cfg.guidance_drop == "interface" and guidance_pair_keep is None:
                raise ValueError("guidance_drop='interface' needs guidance_pair_keep (interface_pair_keep(asym_id))")
            terms = (GuidanceTerm(cfg.guidance_scale, guidance_pair_keep, cfg.guidance_sigma_range),)
        if cfg.skip_amp_sample:
            embeddings, ref_pos, ref_charge, seq_mask, rel_feat = (
                upcast_fp32(t) for t in (embeddings, ref_pos, ref_charge, seq_mask, rel_feat)
            )
            ctx = torch.amp.autocast(device_type=ref_mask.device.type, enabled=False)
        else:
            ctx = nullcontext()
        with ctx:
            return self._sample_impl(
                embeddings, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, seq_mask, rel_feat,
                generator, ref_space_uid, terms, tuple(restraints), restraint_weight, restraint_rigid,
                restraint_max_step, restraint_after_step, restraint_after_sigma,
            )  # fmt: skip

    def _sample_impl(self, embeddings, ref_pos, ref_mask, ref_element, ref_charge, ref_atom_name_chars, seq_mask,
                     rel_feat, generator, ref_space_uid, guidance_terms, restraints, restraint_weight,
                     restraint_rigid, restraint_max_step, restraint_after_step, restraint_after_sigma):  # fmt: skip
        from . import restraints as rst

        cfg = self.cfg
        batched = ref_pos.dim() == 4
        N, M = ref_mask.shape[-2:]
        dev = ref_mask.device
        S = cfg.num_samples
        inputs = dict(
            embeddings={k: _batched(v, batched) for k, v in embeddings.items()},
            ref_pos=_batched(ref_pos, batched), ref_mask=_batched(ref_mask, batched),
            ref_element=_batched(ref_element, batched), ref_charge=_batched(ref_charge, batched),
            ref_atom_name_chars=_batched(ref_atom_name_chars, batched), seq_mask=_batched(seq_mask, batched),
            rel_feat=_batched(rel_feat, batched), ref_space_uid=_batched(ref_space_uid, batched),
        )  # fmt: skip
        B = inputs["ref_pos"].shape[0]
        sigmas = noise_schedule(torch.linspace(0, 1, cfg.steps + 1, device=dev), cfg.sigma_data, cfg.smin, cfg.smax,
                                cfg.noise_p)  # fmt: skip
        gammas = torch.where(sigmas[1:] > cfg.gamma_min, cfg.gamma_0, 0.0)
        sig_hat_all = sigmas[:-1] * (1 + gammas)
        # one host read of the whole schedule; the loop below never syncs on it again
        sig_host, sig_hat_host = sigmas.tolist(), sig_hat_all.tolist()

        # noise is drawn at the unpadded token count so bucket padding does not change the sample
        any_tok = inputs["seq_mask"].reshape(-1, N).bool().any(dim=0)
        nz = torch.nonzero(any_tok)
        n_real = int(nz[-1].item()) + 1 if nz.numel() > 0 else N

        def randn_tokens():
            shape = (B, S) if batched else (S,)
            t = torch.randn(*shape, n_real, M, 3, device=dev, generator=generator)
            t = t if n_real == N else F.pad(t, (0, 0, 0, 0, 0, N - n_real))
            return t if batched else t.unsqueeze(0)

        positions = randn_tokens() * sig_host[0]
        aug_mask = inputs["ref_mask"].bool()
        static = self.compute_static(**inputs)
        uncond = []
        for term in guidance_terms:
            if term.pair_keep is not None:
                emb_u = mask_trunk_pair(inputs["embeddings"], _batched(term.pair_keep, batched), self.null_pair)
                static_u = self.compute_static(**{**inputs, "embeddings": emb_u})
            else:
                static_u = self.compute_static(**inputs, use_conditioning=False)
            lo, hi = term.sigma_range or (float("-inf"), float("inf"))
            uncond.append((term.scale, static_u, lo, hi))

        atom_mask_b = aug_mask if batched else aug_mask[0]
        statics = [static] + [u[1] for u in uncond]
        if denoise_graph.enabled(positions) and cfg.steps > 4 and len(statics) == 1:
            graphs = self.__dict__.setdefault("_denoiser_graphs", denoise_graph.DenoiserGraphs())
            nl0 = positions.new_full((B, 1), sig_hat_host[0])
            denoisers = [graphs.get(self._denoise_core, positions, nl0, st) for st in statics]
        else:
            denoisers = [lambda p, n, st=st: self._denoise_core(p, n, st) for st in statics]
        for step in range(cfg.steps):
            s_prev, s_next, s_hat = sig_host[step], sig_host[step + 1], sig_hat_host[step]
            positions = augment(positions, aug_mask, generator)
            noise_scale = cfg.noise_scale * max(s_hat**2 - s_prev**2, 0.0) ** 0.5
            pos_hat = positions + noise_scale * randn_tokens()
            nl = pos_hat.new_full((B, 1), s_hat)
            den_c = denoisers[0](pos_hat, nl)
            denoised = den_c
            for ui, (w, static_u, lo, hi) in enumerate(uncond):
                if lo <= s_hat <= hi:
                    denoised = denoised + (w - 1.0) * (den_c - denoisers[ui + 1](pos_hat, nl))
            steer = not restraint_after_step or s_hat < restraint_after_sigma
            if restraints and restraint_weight and steer:
                denoised = rst.steer(denoised, atom_mask_b, restraints, s_hat, cfg.sigma_data, restraint_weight,
                                     restraint_rigid, restraint_max_step, batched)  # fmt: skip
            positions = pos_hat + cfg.step_scale * (s_next - s_hat) * (pos_hat - denoised) / s_hat
            last = step == cfg.steps - 1
            if restraints and restraint_weight and restraint_after_step and s_hat >= restraint_after_sigma and not last:
                positions = rst.steer(positions, atom_mask_b, restraints, s_hat, cfg.sigma_data, restraint_weight,
                                      restraint_rigid, restraint_max_step, batched)  # fmt: skip
        mask = inputs["ref_mask"].unsqueeze(1).expand(B, S, N, M)
        if not batched:
            positions, mask = positions[0], mask[0]
        return {"atom_positions": positions, "mask": mask}

    # ---- training rollout ----
    def sample_training(self, gt_positions, gt_mask, embeddings, ref_pos, ref_mask, ref_element, ref_charge,
                        ref_atom_name_chars, seq_mask, rel_feat, num_samples=1, static=None, ref_space_uid=None,
                        clean_mask=None, use_conditioning=True):  # fmt: skip
        """Augment GT, add noise at sampled levels, denoise once (reference: diffusion.py:1623-1775).

        Returns ``(gt_augmented, denoised, noise_levels)`` of shapes ``[B?, S, N, M, 3]`` (x2) and ``[B?, S]``.
        """
        cfg = self.cfg
        if cfg.skip_amp_sample_training:
            gt_positions, embeddings, ref_pos, ref_charge, seq_mask, rel_feat = (
                upcast_fp32(t) for t in (gt_positions, embeddings, ref_pos, ref_charge, seq_mask, rel_feat)
            )
            ctx = torch.amp.autocast(device_type=gt_positions.device.type, enabled=False)
        else:
            ctx = nullcontext()
        batched = gt_positions.dim() == 4
        with ctx:
            gt_b, mask_b = _batched(gt_positions, batched), _batched(gt_mask, batched)
            B, dev = gt_b.shape[0], gt_b.device
            S = num_samples
            gt_aug = augment(gt_b.unsqueeze(1).expand(B, S, *gt_b.shape[1:]), mask_b.bool(), None)
            import math

            ln_sd = math.log(cfg.sigma_data)
            log_sigma = ln_sd + cfg.p_mean + cfg.p_std * torch.randn(B, S, device=dev)
            if cfg.sigma_mix_alpha > 0.0:
                if cfg.sigma_mix_kind == "uniform":
                    lo = math.log(cfg.sigma_data * cfg.sigma_mix_smin)
                    hi = math.log(cfg.sigma_data * cfg.sigma_mix_smax)
                    log_mix = lo + torch.rand(B, S, device=dev) * (hi - lo)
                else:
                    log_mix = ln_sd + cfg.sigma_mix_p_mean + cfg.sigma_mix_p_std * torch.randn(B, S, device=dev)
                log_sigma = torch.where(torch.rand(B, S, device=dev) < cfg.sigma_mix_alpha, log_mix, log_sigma)
            noise_levels = log_sigma.exp()
            if cfg.clamp_train_sigma:
                noise_levels = noise_levels.clamp(min=cfg.train_sigma_min)
            noisy = gt_aug + torch.randn_like(gt_aug) * noise_levels[:, :, None, None, None]
            if clean_mask is not None:
                cm = _batched(clean_mask, batched)[:, :, :, None, None]
                noisy = torch.where(cm, gt_aug, noisy)
            if static is None:
                static = self.compute_static(
                    {k: _batched(v, batched) for k, v in embeddings.items()}, _batched(ref_pos, batched),
                    _batched(ref_mask, batched), _batched(ref_element, batched), _batched(ref_charge, batched),
                    _batched(ref_atom_name_chars, batched), _batched(seq_mask, batched), _batched(rel_feat, batched),
                    _batched(ref_space_uid, batched), use_conditioning,
                )  # fmt: skip
            denoised = self._denoise_samples(noisy, noise_levels, static)
        if not batched:
            gt_aug, denoised, noise_levels = gt_aug[0], denoised[0], noise_levels[0]
        return gt_aug, denoised, noise_levels
