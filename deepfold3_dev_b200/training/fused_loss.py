"""Linear projection + cross-entropy evaluated in row blocks, so ``[S, N, N, bins]`` logits never exist at once.

Same contract as the reference (training/fused_loss.py:20-351): the forward
walks the pair tensor in blocks of ``chunk_n`` rows, computes the block's
logits, loss and the gradient with respect to features and weight, and
keeps only the gradients; backward scales them by the incoming gradient.
``symmetrize`` adds the transposed half-logits (distogram and PDE heads).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from . import losses as L


class _BlockedLinearCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, features, weight, target, mask, chunk_n: int, symmetrize: bool, per_sample: bool):
        S, N, _, H = features.shape
        C = weight.shape[0]
        dev = features.device
        w32 = weight.float()
        if mask is None:
            mask = torch.ones(S, N, N, device=dev)
        mask = mask.float().expand(S, N, N)
        # per_sample: each sample's sum is divided by its own count and the S results are averaged
        denom = mask.sum(dim=(1, 2)).clamp(min=1) * S if per_sample else mask.sum().clamp(min=1).expand(S)
        scale = (1.0 / denom).view(S, 1, 1)
        loss = torch.zeros((), device=dev)
        g_feat = torch.zeros_like(features)
        g_w = torch.zeros(C, H, device=dev)
        for lo in range(0, N, chunk_n):
            hi = min(lo + chunk_n, N)
            rows = features[:, lo:hi].float()
            logits = rows @ w32.T
            if symmetrize:
                cols = features[:, :, lo:hi].float()
                logits = logits + (cols @ w32.T).transpose(1, 2)
            lp = F.log_softmax(logits, dim=-1)
            tgt = target[:, lo:hi].long().unsqueeze(-1)
            m = mask[:, lo:hi] * scale
            loss = loss + (-lp.gather(-1, tgt).squeeze(-1) * m).sum()
            g = lp.exp()
            g.scatter_add_(-1, tgt, torch.full_like(tgt, -1, dtype=g.dtype))
            g = g * m.unsqueeze(-1)
            g_feat[:, lo:hi] += (g @ w32).to(features.dtype)
            g_w += g.reshape(-1, C).T @ rows.reshape(-1, H)
            if symmetrize:
                gt = g.transpose(1, 2)
                g_feat[:, :, lo:hi] += (gt @ w32).to(features.dtype)
                g_w += gt.reshape(-1, C).T @ cols.reshape(-1, H)
        ctx.save_for_backward(g_feat, g_w.to(weight.dtype))
        ctx.flags = (features.requires_grad, weight.requires_grad)
        return loss

    @staticmethod
    def backward(ctx, grad_out):
        g_feat, g_w = ctx.saved_tensors
        need_f, need_w = ctx.flags
        return (g_feat * grad_out if need_f else None, g_w * grad_out if need_w else None, None, None, None, None, None)


def blocked_linear_ce(features, weight, target, mask=None, chunk_n: int = 32, symmetrize: bool = False,
                      per_sample: bool = False):  # fmt: skip
    """Mean CE of ``features @ weight.T`` (optionally symmetrised) against ``target`` ``[S, N, N]`` under ``mask``."""
    return _BlockedLinearCE.apply(features, weight, target, mask, chunk_n, symmetrize, per_sample)


def _distance_bins(x, first, last, bins):
    d = torch.cdist(x, x)
    return torch.bucketize(d, torch.linspace(first, last, bins - 1, device=d.device))


def distogram_loss_fused(pair, weight, gt_positions, token_mask, chunk_n=32, first_break=2.3125,
                         last_break=21.6875, num_bins=64):  # fmt: skip
    """Distogram CE from pair activations ``[B?, N, N, C]`` and the head weight, logits symmetrised."""
    feats = pair if pair.dim() == 4 else pair.unsqueeze(0)
    target = _distance_bins(gt_positions, first_break, last_break, num_bins).unsqueeze(0)
    return blocked_linear_ce(feats, weight, target, L._offdiag_pair_mask(token_mask).unsqueeze(0), chunk_n, True)


@torch.no_grad()
def distogram_entropy_fused(pair, weight, token_mask, chunk_n=32):
    feats = pair if pair.dim() == 4 else pair.unsqueeze(0)
    pm = L._offdiag_pair_mask(token_mask)
    N = pm.shape[0]
    w32 = weight.float()
    total = torch.zeros((), device=pair.device)
    for lo in range(0, N, chunk_n):
        hi = min(lo + chunk_n, N)
        logits = feats[0, lo:hi].float() @ w32.T + (feats[0, :, lo:hi].float() @ w32.T).transpose(0, 1)
        lp = F.log_softmax(logits, dim=-1)
        total = total + (-(lp.exp() * lp).sum(-1) * pm[lo:hi]).sum()
    return total / pm.sum().clamp(min=1)


def pde_loss_fused(features, weight, pred_pos, gt_pos, token_mask, chunk_n=32, max_error=31.0, num_bins=64):
    err = (torch.cdist(pred_pos, pred_pos) - torch.cdist(gt_pos, gt_pos).unsqueeze(0)).abs()
    target = torch.bucketize(err, torch.linspace(0, max_error, num_bins - 1, device=err.device)).clamp(max=num_bins - 1)
    S = features.shape[0]
    mask = L._offdiag_pair_mask(token_mask).unsqueeze(0).expand(S, -1, -1)
    return blocked_linear_ce(features, weight, target, mask, chunk_n, True)


def pae_loss_fused(features, weight, pred_rep, pred_frames, gt_rep, gt_frames, pae_mask, chunk_n=32, num_bins=64,
                   max_error_bin=31.0, angle_threshold=25.0, frame_error=None):  # fmt: skip
    if frame_error is None:
        frame_error = L.frame_aligned_error(pred_rep, pred_frames, gt_rep, gt_frames, angle_threshold)
    err, pred_ok, gt_ok = frame_error
    edges = torch.linspace(0, max_error_bin, num_bins - 1, device=err.device)
    target = torch.bucketize(err, edges).clamp(max=num_bins - 1)
    mask = pae_mask.unsqueeze(0) * pred_ok.float().unsqueeze(-1) * gt_ok.float()[None, :, None]
    return blocked_linear_ce(features, weight, target, mask, chunk_n, False, per_sample=True)
