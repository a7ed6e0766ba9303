"""Optional structure losses: chirality, backbone chirality, FAPE, shape complementarity.

All are off in the default recipe (their ``alpha_*`` weights are 0); reference:
training/loss.py:392-755 (shape complementarity), :1531-1798 (FAPE), :2045-2320 (chirality).
Everything here runs in fp32 with autocast disabled: cross products and frame construction are
noise-sensitive in bf16.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _fp32(device_type):
    return torch.amp.autocast(device_type=device_type, enabled=False)


def _frame_axes(a, b, c):
    """Orthonormal axes (e1, e2, e3) of the frame with origin ``b`` built from the bisector of (a - b, c - b)."""
    w1 = F.normalize(a - b, dim=-1, eps=1e-8)
    w2 = F.normalize(c - b, dim=-1, eps=1e-8)
    e1 = F.normalize(w1 + w2, dim=-1, eps=1e-8)
    e2 = F.normalize(w2 - w1, dim=-1, eps=1e-8)
    return e1, e2, torch.cross(e1, e2, dim=-1)


def _probe_height(pred_pos, frame_token_index, frame_atom_index, chirality_atom_idx):
    pred32 = pred_pos.float()
    n = pred32.shape[1]
    fr = pred32[:, frame_token_index, frame_atom_index]  # [S, N, 3, 3]
    a, b, c = fr[..., 0, :], fr[..., 1, :], fr[..., 2, :]
    probe = pred32[:, torch.arange(n, device=pred32.device), chirality_atom_idx]
    return ((probe - b) * _frame_axes(a, b, c)[2]).sum(-1)  # [S, N]


def chirality_loss(pred_pos, frame_token_index, frame_atom_index, chirality_atom_idx, chirality_target):
    """Mean over marked residues of ``(height of the probe atom above the frame plane - signed target)^2``."""
    target = chirality_target.float()
    valid = (target.abs() > 0).float()
    if float(valid.sum()) == 0:
        return pred_pos.new_zeros(())
    with _fp32(pred_pos.device.type):
        z = _probe_height(pred_pos, frame_token_index, frame_atom_index, chirality_atom_idx)
        mask = valid.unsqueeze(0).expand_as(z)
        loss = (((z - target.unsqueeze(0)) ** 2) * mask).sum() / mask.sum().clamp(min=1)
    return loss.to(pred_pos.dtype)


@torch.no_grad()
def chirality_violation_rates(pred_pos, frame_token_index, frame_atom_index, chirality_atom_idx, chirality_target,
                              margin: float = 0.5) -> dict:  # fmt: skip
    target = chirality_target.float()
    valid = (target.abs() > 0).float()
    if float(valid.sum()) == 0:
        z = pred_pos.new_zeros(())
        return {"chirality_mirror_rate": z, "chirality_ambiguous_rate": z, "chirality_correctness_mean": z}
    with _fp32(pred_pos.device.type):
        corr = _probe_height(pred_pos, frame_token_index, frame_atom_index, chirality_atom_idx) * target.unsqueeze(0)
        mask = valid.unsqueeze(0).expand_as(corr)
        n = mask.sum().clamp(min=1)
        return {"chirality_mirror_rate": ((corr < 0).float() * mask).sum() / n,
                "chirality_ambiguous_rate": ((corr < margin).float() * mask).sum() / n,
                "chirality_correctness_mean": (corr * mask).sum() / n}  # fmt: skip


def _dihedral(p1, p2, p3, p4, eps: float = 1e-8):
    b1, b2, b3 = p2 - p1, p3 - p2, p4 - p3
    b2n = b2 / torch.linalg.norm(b2, dim=-1, keepdim=True).clamp(min=eps)
    n1, n2 = torch.cross(b1, b2, dim=-1), torch.cross(b2, b3, dim=-1)
    m1 = torch.cross(n1, b2n, dim=-1)
    return torch.atan2((m1 * n2).sum(-1), (n1 * n2).sum(-1))


def backbone_chirality_loss(pred_pos, gt_pos, atom_mask, seq_mask, asym_id, mol_type, ca_slot: int = 1):
    """``(sin of the CA pseudo-dihedral - sin of the true one)^2`` over runs of four protein residues of one chain."""
    n = pred_pos.shape[1]
    if n < 4:
        return pred_pos.new_zeros(())
    valid = seq_mask.bool() & (mol_type == 0) & (atom_mask[:, ca_slot] > 0)
    same = (asym_id[:-3] == asym_id[1:-2]) & (asym_id[1:-2] == asym_id[2:-1]) & (asym_id[2:-1] == asym_id[3:])
    quad = valid[:-3] & valid[1:-2] & valid[2:-1] & valid[3:] & same
    if not bool(quad.any()):
        return pred_pos.new_zeros(())
    with _fp32(pred_pos.device.type):
        p = pred_pos.float()[:, :, ca_slot]
        g = gt_pos.float()[:, ca_slot]
        dp = _dihedral(p[:, :-3], p[:, 1:-2], p[:, 2:-1], p[:, 3:])
        with torch.no_grad():
            dg = _dihedral(g[:-3], g[1:-2], g[2:-1], g[3:])
        per = (torch.sin(dp) - torch.sin(dg).unsqueeze(0)) ** 2
        mask = quad.float().unsqueeze(0).expand_as(per)
        loss = (per * mask).sum() / mask.sum().clamp(min=1)
    return loss.to(pred_pos.dtype)


def _frames(pos, frame_token_index, frame_atom_index):
    fr = pos[..., frame_token_index, frame_atom_index, :]  # [..., N, 3, 3]
    a, b, c = fr[..., 0, :], fr[..., 1, :], fr[..., 2, :]
    return torch.stack(_frame_axes(a, b, c), dim=-2), b  # rotation rows = axes, origin


def fape_loss(pred_pos, gt_pos, fape_token_index, fape_atom_index, fape_atom_mask, frame_atom_index, frame_token_index,
              pair_mask, clip_distance: float = 10.0, normalize: bool = True, asym_id=None,
              clip_distance_inter: float = 30.0, mode: str = "pooled", chunk_size: int = 0, eps: float = 1e-4):  # fmt: skip
    """Frame-aligned point error over (frame i, token j, slot k); returns ``(intra_or_pooled, inter)`` scalars.

    ``pair_mask [N, N]`` marks valid (frame token, point token) pairs. ``mode``: ``pooled`` clamps every pair at
    ``clip_distance``; ``both`` / ``intra`` / ``inter`` split pairs by chain and clamp cross-chain pairs at
    ``clip_distance_inter``.
    """
    if mode != "pooled" and asym_id is None:
        raise ValueError("fape_loss: asym_id is required unless mode='pooled'")
    with _fp32(pred_pos.device.type):
        p, g = pred_pos.float(), gt_pos.float()
        S, N = p.shape[0], p.shape[1]
        Rp, tp = _frames(p, frame_token_index, frame_atom_index)  # [S, N, 3, 3], [S, N, 3]
        Rg, tg = _frames(g, frame_token_index, frame_atom_index)
        xp = p[:, fape_token_index, fape_atom_index]  # [S, N, K, 3]
        xg = g[fape_token_index, fape_atom_index]  # [N, K, 3]
        w = pair_mask.float()[:, :, None] * fape_atom_mask.float()[None, :, :]  # [Ni, Nj, K]
        same = None if asym_id is None else (asym_id[:, None] == asym_id[None, :]).float()[:, :, None]
        sums = {"intra": p.new_zeros(S), "inter": p.new_zeros(S)}
        cnts = {"intra": p.new_zeros(()), "inter": p.new_zeros(())}
        step = chunk_size if chunk_size and chunk_size > 0 else N
        for s0 in range(0, N, step):
            sl = slice(s0, min(N, s0 + step))
            dp = xp[:, None, :, :, :] - tp[:, sl, None, None, :]  # [S, i, j, K, 3]
            dg = xg[None, :, :, :] - tg[sl, None, None, :]  # [i, j, K, 3]
            lp = torch.einsum("siac,sijkc->sijka", Rp[:, sl], dp)
            lg = torch.einsum("iac,ijkc->ijka", Rg[sl], dg)
            d = torch.sqrt(((lp - lg.unsqueeze(0)) ** 2).sum(-1) + eps)  # [S, i, j, K]
            wc = w[sl]
            if mode == "pooled":
                e = d.clamp(max=clip_distance) / (clip_distance if normalize else 1.0)
                sums["intra"] = sums["intra"] + (e * wc).sum((1, 2, 3))
                cnts["intra"] = cnts["intra"] + wc.sum()
            else:
                for name, sel, clip in (("intra", same[sl], clip_distance), ("inter", 1.0 - same[sl], clip_distance_inter)):
                    e = d.clamp(max=clip) / (clip if normalize else 1.0)
                    sums[name] = sums[name] + (e * wc * sel).sum((1, 2, 3))
                    cnts[name] = cnts[name] + (wc * sel).sum()
        intra = (sums["intra"] / cnts["intra"].clamp(min=1)).mean()
        inter = (sums["inter"] / cnts["inter"].clamp(min=1)).mean()
        if mode == "intra":
            inter = inter * 0
        if mode == "inter":
            intra = intra * 0
    return intra.to(pred_pos.dtype), inter.to(pred_pos.dtype)


def fape_from_features(denoised, gt_pos, atom_mask, gt_seq_mask, frames_gt_present, features, cfg):
    """FAPE of the denoised samples with the frame / point tables of the featuriser; returns ``(fape, fape_inter)``."""
    frames_ok = features["frames_mask"].bool() & gt_seq_mask.bool()
    if frames_gt_present is not None:
        frames_ok = frames_ok & frames_gt_present.bool()
    pts_tok, pts_atom = features["fape_token_index"], features["fape_atom_index"]
    pts_ok = features["fape_atom_mask"].bool() & atom_mask.bool()[pts_tok, pts_atom] & gt_seq_mask.bool()[:, None]
    pair = frames_ok[:, None] & gt_seq_mask.bool()[None, :]
    mode = cfg.fape_mode if cfg.alpha_fape_inter <= 0 or cfg.fape_mode != "pooled" else "both"
    return fape_loss(denoised, gt_pos, pts_tok, pts_atom, pts_ok, features["frame_atom_index"], features["frame_token_index"],
                     pair, cfg.fape_clip_distance, cfg.fape_normalize, features.get("asym_id"), cfg.fape_clip_distance_inter,
                     mode, cfg.fape_chunk_size)  # fmt: skip


# ------------------------------------------------------------------------------------------------
def _interface_profile(centers, asym_id, valid, density_sigma, interface_cutoff, gap_mean, gap_scale, clash_distance,
                       clash_scale, chunk_size):  # fmt: skip
    """Per-token smooth interface descriptors: partner density, gap score, clash score."""
    n = centers.shape[-2]
    dens, gap, clash = [], [], []
    other = (asym_id[:, None] != asym_id[None, :]) & valid[:, None] & valid[None, :]
    for s0 in range(0, n, chunk_size):
        sl = slice(s0, min(n, s0 + chunk_size))
        d = torch.cdist(centers[..., sl, :], centers)  # [..., c, N]
        m = other[sl].float()
        near = torch.sigmoid((interface_cutoff - d) / density_sigma) * m
        dens.append(near.sum(-1))
        gap.append((torch.exp(-(((d - gap_mean) / gap_scale) ** 2)) * m).sum(-1))
        clash.append((F.softplus((clash_distance - d) / clash_scale) * m).sum(-1))
    return torch.cat(dens, -1), torch.cat(gap, -1), torch.cat(clash, -1)


def shape_complementarity_loss(pred_pos, gt_pos, atom_mask, token_to_rep_atom, asym_id, mol_type, seq_mask,
                               sample_weight=None, density_sigma=1.5, interface_cutoff=16.0, gap_mean=6.0, gap_scale=3.0,
                               clash_distance=2.0, clash_scale=0.5, pool_temperature=16.0, normal_strength_min=1e-4,
                               huber_delta=0.01, pair_weight=0.4, token_weight=1.0, global_weight=0.4, chunk_size=128,
                               eps=1e-6):  # fmt: skip
    """Match smooth interface descriptors of the prediction to those of the ground truth.

    For the representative atom of every token three differentiable per-token quantities are formed from the
    distances to tokens of other chains: partner density inside ``interface_cutoff``, a gap score peaked at
    ``gap_mean`` and a clash score below ``clash_distance``. The loss is a Huber distance between predicted and true
    profiles at token level, at chain-pair level (profiles pooled per chain) and globally, plus the predicted
    clash score, weighted ``token_weight / pair_weight / global_weight``. Returns ``(loss, parts)``.
    """
    with _fp32(pred_pos.device.type):
        n = pred_pos.shape[1]
        ar = torch.arange(n, device=pred_pos.device)
        valid = seq_mask.bool() & (atom_mask[ar, token_to_rep_atom] > 0)
        if len(torch.unique(asym_id[valid])) < 2:
            z = pred_pos.new_zeros(())
            return z, {"shape_comp_token": z, "shape_comp_pair": z, "shape_comp_global": z, "shape_comp_clash": z}
        cp = pred_pos.float()[:, ar, token_to_rep_atom]  # [S, N, 3]
        cg = gt_pos.float()[ar, token_to_rep_atom]  # [N, 3]
        args = (asym_id, valid, density_sigma, interface_cutoff, gap_mean, gap_scale, clash_distance, clash_scale, chunk_size)
        dp, gp, kp = _interface_profile(cp, *args)
        with torch.no_grad():
            dg, gg, _ = _interface_profile(cg, *args)
        w = torch.ones(cp.shape[0], device=cp.device) if sample_weight is None else sample_weight.float()
        w = w / w.sum().clamp(min=eps)
        vm = valid.float()

        def huber(a, b):
            return F.huber_loss(a, b.expand_as(a), reduction="none", delta=huber_delta) / huber_delta

        scale = 1.0 / pool_temperature
        tok = ((huber(dp * scale, dg * scale) + huber(gp * scale, gg * scale)) * vm).sum(-1) / vm.sum().clamp(min=1)
        ids = asym_id.long()
        k = int(ids.max()) + 1
        onehot = F.one_hot(ids, k).float() * vm[:, None]
        pool = lambda t: (t.unsqueeze(-1) * onehot).sum(-2) / onehot.sum(0).clamp(min=1)  # noqa: E731
        pair = (huber(pool(dp) * scale, pool(dg) * scale) + huber(pool(gp) * scale, pool(gg) * scale)).mean(-1)
        glob = huber((dp * vm).sum(-1, keepdim=True) * scale / n, (dg * vm).sum(-1, keepdim=True) * scale / n).squeeze(-1)
        clash = (kp * vm).sum(-1) / vm.sum().clamp(min=1)
        parts = {"shape_comp_token": (tok * w).sum(), "shape_comp_pair": (pair * w).sum(),
                 "shape_comp_global": (glob * w).sum(), "shape_comp_clash": (clash * w).sum()}  # fmt: skip
        loss = (token_weight * parts["shape_comp_token"] + pair_weight * parts["shape_comp_pair"]
                + global_weight * parts["shape_comp_global"] + max(normal_strength_min, 0.0) * 0 + parts["shape_comp_clash"])  # fmt: skip
    return loss.to(pred_pos.dtype), parts


def shape_comp_kwargs(cfg) -> dict:
    return dict(density_sigma=cfg.shape_comp_density_sigma, interface_cutoff=cfg.shape_comp_interface_cutoff,
                gap_mean=cfg.shape_comp_gap_mean, gap_scale=cfg.shape_comp_gap_scale,
                clash_distance=cfg.shape_comp_clash_distance, clash_scale=cfg.shape_comp_clash_scale,
                pool_temperature=cfg.shape_comp_pool_temperature, normal_strength_min=cfg.shape_comp_normal_strength_min,
                huber_delta=cfg.shape_comp_huber_delta, pair_weight=cfg.shape_comp_pair_weight,
                token_weight=cfg.shape_comp_token_weight, global_weight=cfg.shape_comp_global_weight,
                chunk_size=cfg.shape_comp_chunk_size)  # fmt: skip


def shape_comp_sample_weight(cfg, noise_levels: torch.Tensor):
    """Samples noisier than ``shape_comp_sigma_max`` do not contribute (their interfaces are not formed yet)."""
    if cfg.shape_comp_sigma_max is None:
        return None
    return (noise_levels.reshape(-1) <= cfg.shape_comp_sigma_max).float()
