"""Training losses (part 1): alignment, diffusion MSE, smooth LDDT, distogram, confidence heads, bonds.

Reference: training/loss.py:31-2046. Every function takes one example
(no batch axis) and a leading sample axis ``S`` where it applies.
"""

from __future__ import annotations

import math
from contextlib import nullcontext

import torch
import torch.nn.functional as F

from ..data import symmetry as sym

MASK_FIXED = "fixed"
MASK_LOSS_WEIGHT = "loss_weight"


# --------------------------------------------------------------------------- geometry helpers
def weighted_rigid_align(gt_pos, pred_pos, weights, eps: float = 1e-6, stop_gradient: bool = True):
    """Rotate + translate ``gt_pos`` ``[..., K, 3]`` onto ``pred_pos`` by weighted Kabsch, in fp32.

    With ``stop_gradient`` (AF3 default) the result is a constant target.
    """
    out_dtype = pred_pos.dtype
    ctx = torch.no_grad() if stop_gradient else nullcontext()
    with ctx, torch.amp.autocast(device_type=gt_pos.device.type, enabled=False):
        g, p, w = gt_pos.float(), pred_pos.float(), weights.float()
        w = w.expand(g.shape[:-1]).unsqueeze(-1)
        wsum = w.sum(dim=-2, keepdim=True).clamp(min=eps)
        g_mu, p_mu = (g * w).sum(-2, keepdim=True) / wsum, (p * w).sum(-2, keepdim=True) / wsum
        gc, pc = g - g_mu, p - p_mu
        u, _, vh = torch.linalg.svd(torch.matmul((gc * w).transpose(-2, -1), pc))
        v, ut = vh.transpose(-2, -1), u.transpose(-2, -1)
        sign = torch.sign(torch.linalg.det(torch.matmul(v, ut)))
        fix = torch.diag_embed(torch.stack([torch.ones_like(sign), torch.ones_like(sign), sign], dim=-1))
        rot = torch.matmul(v, torch.matmul(fix, ut))
        aligned = torch.matmul(gc, rot.transpose(-2, -1)) + p_mu
    return (aligned.detach() if stop_gradient else aligned).to(out_dtype)


class _SafeNorm(torch.autograd.Function):
    """``|diff|`` with backward ``diff / sqrt(|diff|^2 + eps)``: finite where two atoms coincide."""

    @staticmethod
    def forward(ctx, diff, eps):
        d = torch.linalg.vector_norm(diff, dim=-1)
        ctx.save_for_backward(diff, d)
        ctx.eps = eps
        return d

    @staticmethod
    def backward(ctx, grad):
        diff, d = ctx.saved_tensors
        return (grad / torch.sqrt(d * d + ctx.eps)).unsqueeze(-1) * diff, None


def safe_norm(diff, eps: float = 1e-6):
    return _SafeNorm.apply(diff, eps)


class _PairDifference(torch.autograd.Function):
    """``x[pi] - x[pj]`` for row lists ``pi`` (ascending) and ``pj`` into ``x`` ``[A, F]``.

    The backward of plain advanced indexing is an ``index_put`` with accumulation, which sorts the index list on every
    call (9 ms per list for 1.4 M pairs x 48 samples on a B200). Here both gradients are segment sums: ``pi`` is already
    grouped, ``pj`` is grouped by a permutation computed once per call on the index list alone. No atomics, so the result
    does not depend on scheduling.
    """

    @staticmethod
    def forward(ctx, x, pi, pj):
        ctx.save_for_backward(pi, pj)
        ctx.rows = x.shape[0]
        return x.index_select(0, pi) - x.index_select(0, pj)

    @staticmethod
    def backward(ctx, grad):
        pi, pj = ctx.saved_tensors
        grad = grad.contiguous()
        gi = torch.segment_reduce(grad, "sum", lengths=torch.bincount(pi, minlength=ctx.rows), axis=0, unsafe=True)
        order = torch.argsort(pj, stable=True)
        gj = torch.segment_reduce(grad.index_select(0, order), "sum", lengths=torch.bincount(pj, minlength=ctx.rows), axis=0, unsafe=True)
        return gi - gj, None, None


def express_coordinates_in_frame(rep_pos, frame_pos, eps: float = 1e-8):
    """``out[i, j] = R_i^T (rep[j] - b_i)`` with the frame of token ``i`` built from atoms ``(a, b, c)`` (AF3 Alg. 29)."""
    out_dtype = rep_pos.dtype
    rep, fr = rep_pos.float(), frame_pos.float()
    a, b, c = fr[..., 0, :], fr[..., 1, :], fr[..., 2, :]
    w1, w2 = F.normalize(a - b, dim=-1, eps=eps), F.normalize(c - b, dim=-1, eps=eps)
    e1, e2 = F.normalize(w1 + w2, dim=-1, eps=eps), F.normalize(w2 - w1, dim=-1, eps=eps)
    basis = torch.stack([e1, e2, torch.cross(e1, e2, dim=-1)], dim=-2)  # rows = axes
    rel = rep.unsqueeze(-3) - b.unsqueeze(-2)
    return torch.einsum("...iab,...ijb->...ija", basis, rel).to(out_dtype)


def frame_angle_ok(frames, angle_threshold: float = 25.0, eps: float = 1e-8):
    """True where the angle a-b-c lies strictly between ``threshold`` and ``180 - threshold`` degrees."""
    u, v = frames[..., 0, :] - frames[..., 1, :], frames[..., 2, :] - frames[..., 1, :]
    cos = (u * v).sum(-1) / (u.norm(dim=-1).clamp(min=eps) * v.norm(dim=-1).clamp(min=eps))
    lim = math.cos(math.radians(angle_threshold))
    return (cos < lim) & (cos > -lim)


def frame_aligned_error(pred_rep, pred_frames, gt_rep, gt_frames, angle_threshold: float = 25.0):
    """``(error [S, N, N], pred_frame_ok [S, N], gt_frame_ok [N])``."""
    err = (express_coordinates_in_frame(pred_rep, pred_frames) - express_coordinates_in_frame(gt_rep, gt_frames).unsqueeze(0)).norm(dim=-1)
    return err, frame_angle_ok(pred_frames, angle_threshold), frame_angle_ok(gt_frames, angle_threshold)


def tm_score_from_error(error, mask, n_eff: int):
    """TM-like score from a true pairwise frame error ``[S, N, N]`` under ``mask`` (logging only).

    Same kernel ``1 / (1 + (d/d0)^2)``, ``d0 = 1.24 (max(n, 19) - 15)^(1/3) - 1.8``, row-normalised sum and
    maximum over alignment frames as the inference pTM, so the two are on one scale.
    """
    d0 = 1.24 * (max(int(n_eff), 19) - 15) ** (1.0 / 3) - 1.8
    kernel = 1.0 / (1.0 + (error / d0) ** 2)
    norm = mask / mask.sum(dim=-1, keepdim=True).clamp(min=1e-8)
    return (kernel * norm).sum(dim=-1).max(dim=-1).values.mean()


# --------------------------------------------------------------------------- representation regularisers
def _lp_magnitude(x, mask, p: int, what: str):
    if p not in (1, 2):
        raise ValueError(f"{what} must be 1 or 2, got {p}")
    m = mask.float()
    x32 = x.float()
    per = (x32.abs() if p == 1 else x32 * x32).sum(-1) / x.shape[-1]
    return (per * m).sum() / m.sum().clamp(min=1)


def single_repr_reg_loss(single, seq_mask, p: int = 2):
    """Masked mean over tokens of ``sum_c |s|^p / C`` in fp32."""
    return _lp_magnitude(single, seq_mask, p, "single_reg_p")


def pair_repr_reg_loss(pair, pair_mask, p: int = 2):
    return _lp_magnitude(pair, pair_mask, p, "pair_reg_p")


def _log_rms(x, mask, eps: float = 1e-6):
    rms = _lp_magnitude(x, mask, 2, "p").sqrt()
    return rms, (rms + eps).log()


def single_repr_log_rms_loss(single, seq_mask, eps: float = 1e-6):
    """``(rms, log(rms + eps))`` of the single representation over valid tokens."""
    return _log_rms(single, seq_mask, eps)


def pair_repr_log_rms_loss(pair, pair_mask, eps: float = 1e-6):
    return _log_rms(pair, pair_mask, eps)


# --------------------------------------------------------------------------- structure losses
def smooth_lddt_loss(pred_pos, gt_pos, atom_mask, cutoffs=(0.5, 1.0, 2.0, 4.0), inclusion_radius=15.0,
                     nucleotide_inclusion_radius=30.0, min_distance=1e-3, mol_type=None):  # fmt: skip
    """``1 - mean sigmoid(cutoff - |d_pred - d_gt|)`` over ground-truth neighbour pairs (AF3 Alg. 27).

    The neighbour list comes from the ground truth only (radius 30 A when the
    neighbour atom is a nucleotide, else 15 A) and the differentiable part runs
    on that sparse pair list.
    """
    flat = atom_mask.reshape(-1).bool()
    if int(flat.sum()) < 2:
        return pred_pos.new_zeros(())
    S = pred_pos.shape[0]
    gt = gt_pos.reshape(-1, 3)[flat]
    with torch.no_grad():
        d = torch.cdist(gt, gt)
        if mol_type is not None:
            N, M = atom_mask.shape
            mt = mol_type.view(N, 1).expand(N, M).reshape(-1)[flat]
            nuc = (mt == 1) | (mt == 2)
            radius = torch.where(nuc.unsqueeze(0), d.new_tensor(nucleotide_inclusion_radius), d.new_tensor(inclusion_radius))
            pairs = (d < radius) & (d > min_distance)
        else:
            pairs = (d < inclusion_radius) & (d > min_distance)
        pi, pj = pairs.nonzero(as_tuple=True)
        gt_d = d[pi, pj]
        n_pairs = max(pi.numel(), 1)
    del d, pairs
    # atoms become rows, (sample, xyz) the row content: a pair is then one contiguous row read per side
    rows = pred_pos.reshape(S, -1, 3)[:, flat].permute(1, 0, 2).reshape(-1, S * 3)
    diff = _PairDifference.apply(rows, pi, pj).view(-1, S, 3)  # nonzero() lists pairs row-major, so pi ascends
    err = (safe_norm(diff) - gt_d.unsqueeze(-1)).abs()
    score = sum(torch.sigmoid(c - err).sum(0) for c in cutoffs) / (n_pairs * len(cutoffs))
    return (1.0 - score).mean()


def diffusion_mse_loss(pred_pos, gt_pos, atom_mask, noise_levels, sigma_data=16.0, mol_type=None,
                       nucleotide_loss_weight=5.0, ligand_loss_weight=10.0, noised_mask=None, atom_swap_pairs=None,
                       ligand_swap_pairs=None, ligand_perms=None, asym_id=None, entity_id=None, chain_assign=None,
                       atom_perm_pred=None, token_to_rep_atom=None, seq_mask=None, sym_token_index=None,
                       apply_rigid_align=True):  # fmt: skip
    """EDM-weighted MSE between denoised samples and the (aligned, symmetry-resolved) augmented ground truth.

    Atom weights are ``1 + 5 [DNA or RNA] + 10 [ligand]``; the sum is divided by
    3 x the number of supervised atoms; each sample is weighted by
    ``(sigma^2 + sigma_d^2) / (sigma sigma_d)^2`` (reference: loss.py:1004-1205).
    """
    if asym_id is not None and entity_id is not None and gt_pos.dim() >= 4:
        mask_b = atom_mask.bool()
        new = []
        for s in range(gt_pos.shape[0]):
            assign = chain_assign
            if assign is None:
                assign = sym.compute_chain_permutation_tokens(
                    pred_pos[s], gt_pos[s], mask_b, asym_id, entity_id, token_to_rep_atom=token_to_rep_atom,
                    mol_type=mol_type, seq_mask=seq_mask, sym_token_index=sym_token_index,
                )  # fmt: skip
            g, m = sym.apply_chain_permutation_tokens(gt_pos[s], mask_b, asym_id, assign, sym_token_index)
            new.append(g)
            if chain_assign is not None:
                atom_mask = m
        gt_pos = torch.stack(new, dim=0)
    mask = atom_mask.float()
    if mol_type is not None:
        tw = 1.0 + ((mol_type == 1) | (mol_type == 2)).float() * nucleotide_loss_weight
        tw = tw + (mol_type == 3).float() * ligand_loss_weight
        weight = mask * tw.unsqueeze(-1)
    else:
        weight = mask
    if apply_rigid_align:
        S = pred_pos.shape[0]
        gt_pos = weighted_rigid_align(gt_pos.reshape(S, -1, 3), pred_pos.reshape(S, -1, 3), weight.reshape(-1)).reshape_as(pred_pos)
    mb = atom_mask.bool()
    if atom_swap_pairs is not None and len(atom_swap_pairs) > 0:
        gt_pos = sym.apply_token_atom_permutation(pred_pos, gt_pos, mb, atom_swap_pairs)
    if ligand_swap_pairs is not None and len(ligand_swap_pairs) > 0:
        gt_pos = sym.apply_ligand_token_swap(pred_pos, gt_pos, mb, ligand_swap_pairs)
    if ligand_perms is not None and len(ligand_perms) > 0:
        gt_pos = sym.apply_ligand_token_permutation(pred_pos, gt_pos, mb, ligand_perms)
    if noised_mask is None:
        w4 = weight[None, :, :, None]
        n_atoms = mask.sum().clamp(min=1)
    else:
        nm = noised_mask.to(weight.dtype).unsqueeze(-1)
        w4 = (weight.unsqueeze(0) * nm).unsqueeze(-1)
        n_atoms = (mask.unsqueeze(0) * nm).sum(dim=(-2, -1)).clamp(min=1)
    edm = (noise_levels**2 + sigma_data**2) / (noise_levels * sigma_data) ** 2
    per_sample = ((pred_pos - gt_pos) ** 2 * w4).sum(dim=(-3, -2, -1)) / (3.0 * n_atoms)
    return (edm * per_sample).mean()


def bond_loss(pred_pos, bond_atom_indices, gt_distances, bond_mask, sigma_data=16.0, noise_levels=None):
    """Mean squared deviation of bonded-pair distances from their ground-truth values (AF3 eq. 5)."""
    if bond_atom_indices.shape[0] == 0:
        return pred_pos.new_zeros(())
    t1, a1, t2, a2 = (bond_atom_indices[:, k].long() for k in range(4))
    m = bond_mask.float()
    d = torch.sqrt((pred_pos[:, t1, a1] - pred_pos[:, t2, a2]).pow(2).sum(-1) + 1e-6)
    per_sample = ((d - gt_distances.unsqueeze(0)) ** 2 * m).sum(-1) / m.sum().clamp(min=1)
    if noise_levels is not None:
        per_sample = per_sample * (noise_levels**2 + sigma_data**2) / (noise_levels * sigma_data) ** 2
    return per_sample.mean()


# --------------------------------------------------------------------------- cross-entropy heads
def _offdiag_pair_mask(token_mask):
    m = (token_mask.unsqueeze(1) & token_mask.unsqueeze(0)).float()
    return m.fill_diagonal_(0.0)


def _nll(logits, target):
    return -F.log_softmax(logits.float(), dim=-1).gather(-1, target.unsqueeze(-1)).squeeze(-1)


def distogram_loss(logits, gt_positions, token_mask, first_break=2.3125, last_break=21.6875, num_bins=64):
    d = torch.cdist(gt_positions, gt_positions)
    target = torch.bucketize(d, torch.linspace(first_break, last_break, num_bins - 1, device=d.device))
    pm = _offdiag_pair_mask(token_mask)
    return (_nll(logits, target) * pm).sum() / pm.sum().clamp(min=1)


@torch.no_grad()
def distogram_entropy(logits, token_mask):
    pm = _offdiag_pair_mask(token_mask)
    lp = F.log_softmax(logits.float(), dim=-1)
    return (-(lp.exp() * lp).sum(-1) * pm).sum() / pm.sum().clamp(min=1)


def masked_msa_loss(logits, true_msa, bert_mask, eps: float = 1e-8):
    C = logits.shape[-1]
    nll = F.cross_entropy(logits.float().reshape(-1, C), true_msa.long().reshape(-1), reduction="none")
    m = bert_mask.float()
    return (nll.reshape(true_msa.shape) * m).sum() / m.sum().clamp_min(eps)


def per_atom_lddt(pred_pos, gt_pos, atom_mask, cutoffs=(0.5, 1.0, 2.0, 4.0), inclusion_radius=30.0, mol_type=None,
                  rep_idx=None, inclusion_radius_protein=15.0, inclusion_radius_nucleotide=30.0):  # fmt: skip
    """``([S, N, M] LDDT in [0, 1], meaningful)``.

    With ``mol_type`` and ``rep_idx`` the neighbour atoms ``j`` are the
    representative atoms of protein / nucleic tokens (radius 15 / 30 A by the
    type of ``j``); otherwise all resolved atoms within ``inclusion_radius``.
    ``meaningful`` is False when no atom can act as ``i`` or as ``j``.
    """
    S = pred_pos.shape[0]
    N, M = atom_mask.shape
    zero = torch.zeros(S, N, M, device=pred_pos.device, dtype=pred_pos.dtype)
    im = atom_mask.reshape(-1).bool()
    if int(im.sum()) < 1:
        return zero, False
    gt_flat, pred_flat = gt_pos.reshape(-1, 3), pred_pos.reshape(S, -1, 3)
    if mol_type is None or rep_idx is None:
        jm = im
        radius = None
    else:
        is_rep = (torch.arange(M, device=atom_mask.device).unsqueeze(0) == rep_idx.clamp(0, M - 1).unsqueeze(-1))
        is_rep = is_rep & (rep_idx.unsqueeze(-1) >= 0) & (rep_idx.unsqueeze(-1) < M) & atom_mask.bool()
        prot = (mol_type == 0).unsqueeze(-1) & is_rep
        nuc = ((mol_type == 1) | (mol_type == 2)).unsqueeze(-1) & is_rep
        jm = (prot | nuc).reshape(-1)
        if int(jm.sum()) < 1:
            return zero, False
        radius = torch.where(prot.reshape(-1)[jm], inclusion_radius_protein, inclusion_radius_nucleotide)
    gd = torch.cdist(gt_flat[im], gt_flat[jm])
    pm = (gd < (inclusion_radius if radius is None else radius.unsqueeze(0))) & (gd > 1e-3)
    n_pairs = pm.sum(-1).clamp(min=1)
    err = (torch.cdist(pred_flat[:, im], pred_flat[:, jm]) - gd.unsqueeze(0)).abs()
    score = sum(((err < c).float() * pm).sum(-1) / n_pairs for c in cutoffs) / len(cutoffs)
    full = torch.zeros(S, N * M, device=pred_pos.device, dtype=pred_pos.dtype)
    full[:, im] = score.to(full.dtype)
    return full.reshape(S, N, M), True


def plddt_loss(logits, pred_pos, gt_pos, atom_mask, num_bins=50, mol_type=None, rep_idx=None):
    S, N = logits.shape[:2]
    M = atom_mask.shape[-1]
    lr = logits.reshape(S, N, M, num_bins)
    lddt, ok = per_atom_lddt(pred_pos, gt_pos, atom_mask, mol_type=mol_type, rep_idx=rep_idx)
    if not ok:
        return (lr.float().sum() * 0.0).to(logits.dtype)  # term dropped, graph kept connected
    target = (lddt * num_bins).clamp(0, num_bins - 1).long()
    m = atom_mask.float()
    return (_nll(lr, target) * m.unsqueeze(0)).sum() / (m.sum().clamp(min=1) * S)


def _pairwise_binned_loss(logits, error, pair_mask, max_error=31.0, num_bins=64):
    edges = torch.linspace(0, max_error, num_bins - 1, device=logits.device)
    target = torch.bucketize(error, edges).clamp(max=num_bins - 1)
    return (_nll(logits, target) * pair_mask.unsqueeze(0)).sum() / (pair_mask.sum().clamp(min=1) * logits.shape[0])


def pae_loss(logits, pred_rep, pred_frames, gt_rep, gt_frames, pae_mask, num_bins=64, max_error_bin=31.0,
             angle_threshold=25.0, frame_error=None):  # fmt: skip
    if frame_error is None:
        frame_error = frame_aligned_error(pred_rep, pred_frames, gt_rep, gt_frames, angle_threshold)
    error, pred_ok, gt_ok = frame_error
    edges = torch.linspace(0, max_error_bin, num_bins - 1, device=logits.device)
    target = torch.bucketize(error, edges).clamp(max=num_bins - 1)
    mask = pae_mask.unsqueeze(0) * pred_ok.float().unsqueeze(-1) * gt_ok.float()[None, :, None]
    per_sample = (_nll(logits, target) * mask).sum(dim=(-1, -2)) / mask.sum(dim=(-1, -2)).clamp(min=1)
    return per_sample.mean()


def pde_loss(logits, pred_pos, gt_pos, token_mask, max_error=31.0, num_bins=64):
    err = (torch.cdist(pred_pos, pred_pos) - torch.cdist(gt_pos, gt_pos).unsqueeze(0)).abs()
    return _pairwise_binned_loss(logits, err, _offdiag_pair_mask(token_mask), max_error, num_bins)


def exp_resolved_loss(logits, atom_mask, valid_mask, fixed_mask=None):
    """Two-class CE per atom slot; target = resolved mask, or the token's experimental fraction when given."""
    target = atom_mask.float() if fixed_mask is None else fixed_mask.unsqueeze(-1).expand_as(atom_mask).float()
    M = atom_mask.shape[-1]
    lp = F.log_softmax(logits.reshape(*logits.shape[:2], M, 2).float(), dim=-1)
    p = target.unsqueeze(0)
    nll = -(p * lp[..., 1] + (1 - p) * lp[..., 0])
    w = valid_mask.float().unsqueeze(0).expand_as(nll)
    return (nll * w).sum() / w.sum().clamp_min(1.0)
