"""Training objective: symmetry resolution of the ground truth, the diffusion-side loss and the full loss.

Reference: training/loss.py:756-1003 (symmetry), :2474-2742 (``diffusion_only_loss``),
:2743-3419 (``training_loss``). All functions take one example (no batch axis).
"""

from __future__ import annotations

import torch

from ..data import symmetry as sym
from . import losses as L
from .losses import MASK_FIXED, MASK_LOSS_WEIGHT

MOL_NONPOLYMER = 3
_SHAPE_COMP_FEATURES = ("mol_type", "asym_id", "token_to_rep_atom", "seq_mask")


# --------------------------------------------------------------------------- symmetry resolution
def inter_chain_bonds_from_features(features):
    """``(asym_a, asym_b)`` pairs joined by a token bond with a non-polymer end; ``None`` if there are none."""
    bm, asym = features.get("bond_matrix"), features.get("asym_id")
    if bm is None or asym is None or bm.dim() != 3 or bm.shape[0] != asym.shape[0]:
        return None
    with torch.no_grad():
        idx = (bm[..., 0] > 0).nonzero()
    if idx.numel() == 0:
        return None
    a = asym.detach().cpu().numpy()
    mol = features.get("mol_type")
    m = mol.detach().cpu().numpy() if mol is not None else None
    pairs = set()
    for i, j in idx.tolist():
        if i >= j or a[i] == a[j]:
            continue
        if m is not None and m[i] != MOL_NONPOLYMER and m[j] != MOL_NONPOLYMER:
            continue
        pairs.add((int(min(a[i], a[j])), int(max(a[i], a[j]))))
    return sorted(pairs) or None


def chain_perm_from_mini_rollout(pred, features, stability_gate_k: int = 1):
    """Chain assignment from the mini-rollout (shared by all augmented samples); ``{}`` if the K-vote disagrees."""
    mini = pred.get("mini_rollout_pos")
    need = [features.get(k) for k in ("asym_id", "entity_id", "atom_gt_positions", "atom_gt_mask")]
    if mini is None or any(v is None for v in need):
        return None
    asym, ent, gt, mask = need
    vote = pred.get("chain_perm_gate_pos")
    if vote is None or int(stability_gate_k) <= 1:
        vote = mini
    bonds = inter_chain_bonds_from_features(features)

    def assign(s):
        return sym.compute_chain_permutation_tokens(
            vote[s], gt, mask.bool(), asym, ent, token_to_rep_atom=features.get("token_to_rep_atom"),
            mol_type=features.get("mol_type"), seq_mask=features.get("seq_mask"),
            sym_token_index=features.get("sym_token_index"), inter_chain_bonds=bonds,
        )  # fmt: skip

    k = min(int(stability_gate_k), int(vote.shape[0]))
    first = assign(0)
    for s in range(1, k):
        if assign(s) != first:
            return {}
    return first


def resolve_gt_atom_symmetry(ref, features, gt, atom_mask):
    """Relabel symmetric residue / ligand atoms of ``gt`` to best match ``ref`` (the mini-rollout).

    ``ref`` is first aligned onto ``gt`` using the representative atoms only,
    then the swap tables in ``features`` are applied (AF3 supplement 4.2).
    """
    tables = [features.get(k) for k in ("atom_swap_pairs", "ligand_swap_pairs", "ligand_perms")]
    if not any(t is not None and len(t) > 0 for t in tables):
        return gt
    n, m = gt.shape[-3], gt.shape[-2]
    lead = gt.shape[:-3]
    gt_b, ref_b = gt.reshape(-1, n, m, 3), ref.reshape(-1, n, m, 3)
    rep = features.get("token_to_rep_atom")
    if rep is not None:
        w2 = torch.zeros(n, m, device=gt.device, dtype=torch.bool)
        w2[torch.arange(n, device=gt.device), rep.to(gt.device)] = True
        w = (w2 & atom_mask.bool()).reshape(-1).to(gt.dtype)
    else:
        w = atom_mask.reshape(-1).to(gt.dtype)
    with torch.no_grad():
        b = gt_b.shape[0]
        aligned = L.weighted_rigid_align(ref_b.reshape(b, -1, 3).detach(), gt_b.reshape(b, -1, 3), w).reshape(b, n, m, 3)
        mb, out = atom_mask.bool(), gt_b
        if tables[0] is not None and len(tables[0]) > 0:
            out = sym.apply_token_atom_permutation(aligned, out, mb, tables[0])
        if tables[1] is not None and len(tables[1]) > 0:
            out = sym.apply_ligand_token_swap(aligned, out, mb, tables[1])
        if tables[2] is not None and len(tables[2]) > 0:
            out = sym.apply_ligand_token_permutation(aligned, out, mb, tables[2])
    return out.reshape(*lead, n, m, 3)


def resolve_chain_perm_index(pred, features, stability_gate_k: int = 1):
    """``(index, keep)`` reordering GT tokens, or ``(None, None)`` when no chains are exchanged.

    A result stashed by ``forward_training`` in ``features["chain_perm_index"]`` is reused.
    """
    cached = features.get("chain_perm_index")
    if cached is not None:
        return cached, features["chain_perm_keep"]
    assign = chain_perm_from_mini_rollout(pred, features, stability_gate_k)
    asym = features.get("asym_id")
    if assign and asym is not None and not all(int(k) == int(v) for k, v in assign.items()):
        return sym.chain_permutation_index(
            asym, assign, features.get("sym_token_index"), device=features["atom_gt_positions"].device
        )
    return None, None


def permute_gt_for_diffusion(pred, features, stability_gate_k: int = 1):
    """``(gt_positions, gt_mask, index, keep)`` with chain and atom symmetry resolved once from the mini-rollout."""
    gt, mask = features["atom_gt_positions"], features["atom_gt_mask"]
    index, keep = resolve_chain_perm_index(pred, features, stability_gate_k)
    if index is not None:
        gt = gt.index_select(0, index)
        mask = mask.index_select(0, index) & keep.unsqueeze(-1)
    mini = pred.get("mini_rollout_pos")
    if mini is not None:
        gt = resolve_gt_atom_symmetry(mini[0], features, gt, mask)
    return gt, mask, index, keep


def augment_bonds_with_symmetric_pairs(features, gt_pos, atom_mask, idx, gt_d, mask):
    """Append the exchangeable atom pairs to the bond list: their distance is label-invariant (reference: :1980)."""
    dev = gt_pos.device
    rows = []
    asp = features.get("atom_swap_pairs")
    if asp is not None and len(asp) > 0:
        asp = asp.to(dev).long()
        asp = asp[asp[:, 1] != asp[:, 2]]
        if len(asp):
            rows.append(torch.stack([asp[:, 0], asp[:, 1], asp[:, 0], asp[:, 2]], dim=1))
    lsp = features.get("ligand_swap_pairs")
    if lsp is not None and len(lsp) > 0:
        lsp = lsp.to(dev).long()
        lsp = lsp[lsp[:, 0] != lsp[:, 1]]
        if len(lsp):
            z = torch.zeros(lsp.shape[0], dtype=torch.long, device=dev)
            rows.append(torch.stack([lsp[:, 0], z, lsp[:, 1], z], dim=1))
    if idx is not None and idx.shape[0] > 0:
        base = (idx.to(dev).long(), gt_d.to(dev), mask.to(dev).bool())
    else:
        base = (torch.zeros((0, 4), dtype=torch.long, device=dev), torch.zeros(0, device=dev),
                torch.zeros(0, dtype=torch.bool, device=dev))  # fmt: skip
    if not rows:
        return base
    extra = torch.cat(rows, dim=0)
    t1, a1, t2, a2 = extra.unbind(1)
    d = (gt_pos[t1, a1] - gt_pos[t2, a2]).norm(dim=-1)
    ok = atom_mask[t1, a1].bool() & atom_mask[t2, a2].bool()
    return torch.cat([base[0], extra]), torch.cat([base[1], d]), torch.cat([base[2], ok])


def _loss_weight_mask(features):
    m = features.get(f"mask_{MASK_LOSS_WEIGHT}")
    if m is not None and not bool((m < 1.0).any()):
        return None
    return m


# --------------------------------------------------------------------------- diffusion-side terms
def _diffusion_terms(pred, features, cfg, gt_pos, atom_mask, seq_mask, gt_seq_mask, frames_gt_present, detach: bool):
    """Terms computed from the denoised samples. Returns ``(total, components)``.

    Shared by ``diffusion_only_loss`` (per chunk, components detached) and ``training_loss``.
    """
    from . import extra_losses as X

    denoised, gt_aug, sigmas = pred["denoised"], pred["gt_augmented"], pred["noise_levels"]
    pre = features.get("__gt_prepermuted__")
    mini = pred.get("mini_rollout_pos")
    if cfg.diffusion_mse_per_sample_symmetry and not pre:
        kw = {k: features.get(k) for k in ("atom_swap_pairs", "ligand_swap_pairs", "ligand_perms")}
    else:
        if mini is not None and not pre:
            gt_aug = resolve_gt_atom_symmetry(mini[0].unsqueeze(0).expand_as(gt_aug), features, gt_aug, atom_mask)
        kw = {}
    clean = pred.get("diffusion_clean_mask")
    keep = (lambda t: t.detach()) if detach else (lambda t: t)
    comps = {}
    l_mse = L.diffusion_mse_loss(
        denoised, gt_aug, atom_mask, sigmas, mol_type=features.get("mol_type"),
        nucleotide_loss_weight=cfg.nucleotide_loss_weight, ligand_loss_weight=cfg.ligand_loss_weight,
        noised_mask=(~clean.bool()) if clean is not None else None, apply_rigid_align=cfg.use_rigid_align, **kw,
    )  # fmt: skip
    comps["diffusion_mse"] = keep(l_mse)
    total = cfg.alpha_diffusion * l_mse
    if cfg.alpha_smooth_lddt is not None:
        l_lddt = L.smooth_lddt_loss(
            denoised, gt_pos, atom_mask, cutoffs=cfg.lddt_cutoffs, inclusion_radius=cfg.lddt_inclusion_radius,
            nucleotide_inclusion_radius=cfg.lddt_nucleotide_inclusion_radius, min_distance=cfg.lddt_min_distance,
            mol_type=features.get("mol_type"),
        )  # fmt: skip
        comps["smooth_lddt"] = keep(l_lddt)
        total = total + cfg.alpha_diffusion * cfg.alpha_smooth_lddt * l_lddt
    if cfg.alpha_shape_comp > 0 and all(k in features for k in _SHAPE_COMP_FEATURES):
        l_shape, parts = X.shape_complementarity_loss(
            denoised, gt_pos, atom_mask, features["token_to_rep_atom"], features["asym_id"], features["mol_type"],
            seq_mask, sample_weight=X.shape_comp_sample_weight(cfg, sigmas), **X.shape_comp_kwargs(cfg),
        )  # fmt: skip
        comps.update({k: keep(v) for k, v in parts.items()})
        total = total + cfg.alpha_shape_comp * l_shape
    if cfg.alpha_bond > 0 and ("bond_atom_indices" in features or cfg.bond_include_symmetric):
        b_idx, b_gt, b_m = (features.get(k) for k in ("bond_atom_indices", "bond_gt_distances", "bond_loss_mask"))
        if cfg.bond_include_symmetric:
            b_idx, b_gt, b_m = augment_bonds_with_symmetric_pairs(features, gt_pos, atom_mask, b_idx, b_gt, b_m)
        l_bond = L.bond_loss(denoised, b_idx, b_gt, b_m, noise_levels=sigmas)
        comps["bond"] = keep(l_bond)
        total = total + cfg.alpha_diffusion * cfg.alpha_bond * l_bond
    if cfg.alpha_chirality > 0 and "chirality_target" in features:
        args = (denoised, features["frame_token_index"], features["frame_atom_index"], features["chirality_atom_idx"],
                features["chirality_target"])  # fmt: skip
        l_chir = X.chirality_loss(*args)
        comps["chirality"] = keep(l_chir)
        total = total + cfg.alpha_chirality * l_chir
        comps.update({k: keep(v) for k, v in X.chirality_violation_rates(*args, margin=cfg.chirality_margin).items()})
    if cfg.alpha_backbone_chirality > 0 and "mol_type" in features:
        l_bb = X.backbone_chirality_loss(denoised, gt_pos, atom_mask, gt_seq_mask, features["asym_id"], features["mol_type"])
        comps["backbone_chirality"] = keep(l_bb)
        total = total + cfg.alpha_backbone_chirality * l_bb
    fape_keys = ("fape_atom_index", "fape_token_index", "fape_atom_mask", "frame_token_index", "frame_atom_index")
    if (cfg.alpha_fape > 0 or cfg.alpha_fape_inter > 0) and all(k in features for k in fape_keys):
        l_fape, l_inter = X.fape_from_features(denoised, gt_pos, atom_mask, gt_seq_mask, frames_gt_present, features, cfg)
        comps["fape"], comps["fape_inter"] = keep(l_fape), keep(l_inter)
        total = total + cfg.alpha_fape * l_fape + cfg.alpha_fape_inter * l_inter
    return total, comps


def _permuted_gt(pred, features, cfg):
    """Ground truth after chain and atom symmetry resolution: ``(gt_pos, atom_mask, gt_seq_mask, index)``."""
    gt_pos, atom_mask = features["atom_gt_positions"], features["atom_gt_mask"]
    seq_mask = features["seq_mask"].bool()
    index, keep = resolve_chain_perm_index(
        pred, features, stability_gate_k=(cfg.chain_perm_gate_k if cfg.chain_perm_stability_gate else 1)
    )
    gt_seq_mask = seq_mask
    if index is not None:
        gt_pos = gt_pos.index_select(0, index)
        atom_mask = atom_mask.index_select(0, index) & keep.unsqueeze(-1)
        gt_seq_mask = seq_mask & keep
    mini = pred.get("mini_rollout_pos")
    if mini is not None:
        gt_pos = resolve_gt_atom_symmetry(mini[0], features, gt_pos, atom_mask)
    return gt_pos, atom_mask, gt_seq_mask, index


def _frames_gt_present(features, atom_mask, n_tok):
    fa = features.get("frame_atom_index")
    if fa is None:
        return None
    ft = features.get("frame_token_index")
    if ft is None:
        ft = torch.arange(n_tok, device=atom_mask.device).unsqueeze(-1).expand(n_tok, 3)
    return atom_mask.bool()[ft, fa].all(dim=-1)


def diffusion_only_loss(pred, features, cfg):
    """Diffusion-side loss of one chunk of samples: ``(weighted total, detached components)``."""
    gt_pos, atom_mask, gt_seq_mask, index = _permuted_gt(pred, features, cfg)
    if index is not None and not features.get("__gt_prepermuted__"):
        pred = {**pred, "gt_augmented": pred["gt_augmented"].index_select(-3, index)}
    lw = _loss_weight_mask(features)
    if lw is not None:
        atom_mask = atom_mask * lw.unsqueeze(-1)
    present = _frames_gt_present(features, atom_mask, gt_seq_mask.shape[0])
    return _diffusion_terms(pred, features, cfg, gt_pos, atom_mask, gt_seq_mask, gt_seq_mask, present, detach=True)


# --------------------------------------------------------------------------- full loss
def training_loss(pred, features, cfg):
    """Full loss of one example: ``(total, {name: value})`` (reference: loss.py:2743-3419)."""
    seq_mask = features["seq_mask"].bool()
    N = seq_mask.shape[0]
    rep_idx = features.get("token_to_rep_atom")
    center_idx = features.get("token_to_center_atom", rep_idx)
    if center_idx is None:
        center_idx = rep_idx
    gt_pos, atom_mask, gt_seq_mask, index = _permuted_gt(pred, features, cfg)
    mini = pred.get("mini_rollout_pos")
    losses: dict = {}
    anchor = pred["distogram_features"] if "distogram_features" in pred else pred["distogram"]
    total = (anchor.reshape(-1)[0] * 0).float()

    fixed = features.get(f"mask_{MASK_FIXED}")
    if fixed is not None and not fixed.any():
        fixed = None
    lw = _loss_weight_mask(features)
    if lw is not None:
        loss_atom_mask, loss_seq_mask = atom_mask * lw.unsqueeze(-1), gt_seq_mask & (lw >= 0.5)
    else:
        loss_atom_mask, loss_seq_mask = atom_mask, gt_seq_mask
    present = _frames_gt_present(features, atom_mask, N)

    # representation magnitude terms (alpha 0 = observe only)
    for name, alpha, p, tensor, mask, reg, log_reg in (
        ("single", cfg.alpha_single_reg, cfg.single_reg_p, pred.get("single"), seq_mask,
         L.single_repr_reg_loss, L.single_repr_log_rms_loss),
        ("pair", cfg.alpha_pair_reg, cfg.pair_reg_p, pred.get("pair"), None,
         L.pair_repr_reg_loss, L.pair_repr_log_rms_loss),
    ):  # fmt: skip
        if alpha is None or tensor is None:
            continue
        if mask is None:
            mask = features.get("pair_mask")
            if mask is None:
                mask = seq_mask.unsqueeze(-1) & seq_mask.unsqueeze(-2)
        grad_ctx = torch.enable_grad() if alpha > 0 else torch.no_grad()
        with grad_ctx:
            if cfg.reg_form == "log_rms":
                rms, val = log_reg(tensor, mask)
                losses[f"{name}_rms"] = rms
            else:
                val = reg(tensor, mask, p)
                losses[f"{name}_l{p}"] = val
        if alpha > 0:
            total = total + alpha * val

    if "__diffusion_logged__" in pred:
        losses.update(pred["__diffusion_logged__"])
        total = total + pred["__diffusion_total__"]
    elif "denoised" in pred:
        dpred = pred
        if index is not None and not features.get("__gt_prepermuted__"):
            dpred = {**pred, "gt_augmented": pred["gt_augmented"].index_select(-3, index)}
        d_total, comps = _diffusion_terms(
            dpred, features, cfg, gt_pos, loss_atom_mask, seq_mask, gt_seq_mask, present, detach=False
        )
        losses.update(comps)
        total = total + d_total

    ar = torch.arange(N, device=gt_pos.device)
    if rep_idx is not None:
        gt_rep, rep_present = gt_pos[ar, rep_idx], atom_mask[ar, rep_idx].bool()
    else:
        gt_rep, rep_present = gt_pos[:, 1, :], torch.ones(N, dtype=torch.bool, device=gt_pos.device)
    rep_seq_mask = loss_seq_mask & rep_present

    if cfg.alpha_distogram > 0:
        l_d = e_d = None
        if "distogram_features" in pred:
            from . import fused_loss as FL

            l_d = FL.distogram_loss_fused(
                pred["distogram_features"], pred["distogram_weight"], gt_rep, rep_seq_mask, chunk_n=cfg.fused_ce_chunk_n
            )
            if cfg.log_distogram_entropy:
                with torch.no_grad():
                    e_d = FL.distogram_entropy_fused(
                        pred["distogram_features"], pred["distogram_weight"], rep_seq_mask, chunk_n=cfg.fused_ce_chunk_n
                    )
        elif "distogram" in pred:
            l_d = L.distogram_loss(pred["distogram"], gt_rep, rep_seq_mask)
            if cfg.log_distogram_entropy:
                e_d = L.distogram_entropy(pred["distogram"], rep_seq_mask)
        if l_d is not None:
            losses["distogram"] = l_d
            total = total + cfg.alpha_distogram * l_d
        if e_d is not None:
            losses["distogram_entropy"] = e_d

    if "masked_msa_logits" in pred:
        l_m = L.masked_msa_loss(pred["masked_msa_logits"], pred["true_msa"], pred["bert_mask"])
        losses["masked_msa"] = l_m
        total = total + cfg.alpha_masked_msa * l_m

    # true frame-aligned error of the mini-rollout: logged TM scores and the PAE target
    frame_idx, frame_tok, frames_mask = (features.get(k) for k in ("frame_atom_index", "frame_token_index", "frames_mask"))
    if frame_tok is None and frame_idx is not None:
        frame_tok = ar.unsqueeze(-1).expand(N, 3)
    pair_mask_feat = features.get("pair_mask")
    shared_err = None
    if (cfg.log_tm_true or cfg.alpha_pae > 0) and mini is not None and frame_idx is not None and frames_mask is not None:
        with torch.no_grad():
            pred_rep = mini[:, ar, rep_idx] if rep_idx is not None else mini[:, :, 1, :]
            shared_err = L.frame_aligned_error(
                pred_rep, mini[:, frame_tok, frame_idx], gt_rep, gt_pos[frame_tok, frame_idx]
            )
            err, pred_ok, gt_ok = shared_err
            pm = pair_mask_feat if pair_mask_feat is not None else loss_seq_mask.unsqueeze(1) & loss_seq_mask.unsqueeze(0)
            pm = pm.bool() & rep_present.unsqueeze(0) & rep_present.unsqueeze(1)
            fm = frames_mask.bool() if present is None else frames_mask.bool() & present
            mask_s = (fm.unsqueeze(-1) & pm).float().unsqueeze(0) * pred_ok.float().unsqueeze(-1) * gt_ok.float()[None, :, None]
            n_eff = int(rep_seq_mask.sum().item())
            if mask_s.sum() > 0 and n_eff > 0:
                losses["tm_true"] = L.tm_score_from_error(err, mask_s, n_eff)
                asym = features.get("asym_id")
                if asym is not None:
                    cross = mask_s * (asym.unsqueeze(0) != asym.unsqueeze(1)).float().unsqueeze(0)
                    if cross.sum() > 0:
                        losses["itm_true"] = L.tm_score_from_error(err, cross, n_eff)

    dist = features.get("is_distillation")
    if dist is not None and bool(dist.item()):
        losses["total"] = total
        return total, losses

    res = features.get("resolution")
    if res is None:
        conf_ok = torch.ones((), device=gt_pos.device, dtype=gt_pos.dtype)
    else:
        res = res if torch.is_tensor(res) else torch.tensor(res, device=gt_pos.device)
        conf_ok = ((res >= cfg.min_resolution) & (res <= cfg.max_resolution)).to(gt_pos.dtype)

    if cfg.alpha_confidence > 0 and mini is not None:
        w_conf = cfg.alpha_confidence * conf_ok
        if "plddt" in pred:
            losses["plddt"] = L.plddt_loss(
                pred["plddt"], mini, gt_pos, loss_atom_mask, mol_type=features.get("mol_type"), rep_idx=center_idx
            )
            total = total + w_conf * losses["plddt"]
        mini_rep = mini[:, ar, rep_idx] if rep_idx is not None else mini[:, :, 1, :]
        if "pde_features" in pred:
            from . import fused_loss as FL

            losses["pde"] = FL.pde_loss_fused(
                pred["pde_features"], pred["pde_weight"], mini_rep, gt_rep, rep_seq_mask, chunk_n=cfg.fused_ce_chunk_n
            )
            total = total + w_conf * losses["pde"]
        elif "pde" in pred:
            losses["pde"] = L.pde_loss(pred["pde"], mini_rep, gt_rep, rep_seq_mask)
            total = total + w_conf * losses["pde"]
        if "exp_resolved" in pred:
            ref_mask = features.get("ref_mask")
            if ref_mask is None:
                valid = loss_atom_mask
            else:
                valid = ref_mask & gt_seq_mask.unsqueeze(-1)
                if lw is not None:
                    valid = valid * lw.unsqueeze(-1)
            losses["exp_resolved"] = L.exp_resolved_loss(pred["exp_resolved"], loss_atom_mask, valid, fixed)
            total = total + w_conf * losses["exp_resolved"]
        if cfg.alpha_pae > 0 and frame_idx is not None and frames_mask is not None:
            pm = pair_mask_feat
            if pm is None:
                pm = loss_seq_mask.unsqueeze(1) & loss_seq_mask.unsqueeze(0)
            elif lw is not None:
                k = lw >= 0.5
                pm = pm.bool() & k.unsqueeze(1) & k.unsqueeze(0)
            pm = pm.bool() & rep_present.unsqueeze(0) & rep_present.unsqueeze(1)
            fm = frames_mask.bool() if present is None else frames_mask.bool() & present
            pae_mask = (fm.unsqueeze(-1) & pm).float()
            frames = (None, None) if shared_err is not None else (mini[:, frame_tok, frame_idx], gt_pos[frame_tok, frame_idx])
            l_pae = None
            if "pae_features" in pred:
                from . import fused_loss as FL

                l_pae = FL.pae_loss_fused(
                    pred["pae_features"], pred["pae_weight"], mini_rep, frames[0], gt_rep, frames[1], pae_mask,
                    chunk_n=cfg.fused_ce_chunk_n, frame_error=shared_err,
                )  # fmt: skip
            elif "pae" in pred:
                l_pae = L.pae_loss(pred["pae"], mini_rep, frames[0], gt_rep, frames[1], pae_mask, frame_error=shared_err)
            if l_pae is not None:
                losses["pae"] = l_pae
                total = total + w_conf * cfg.alpha_pae * l_pae
    losses["total"] = total
    return total, losses
