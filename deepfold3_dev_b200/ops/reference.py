"""Plain PyTorch statements of every fused op.

These are the CPU path and the numerical oracle the CUDA kernels are tested
against; each function states, in fp32-safe PyTorch, exactly what its kernel
computes. Shapes use ``B`` batch, ``R`` rows (independent attention problems),
``H`` heads, ``N`` tokens, ``D`` head width, ``C`` channels.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

MASK_NEG = 1e9


def layer_norm(x, weight=None, bias=None, eps: float = 1e-5):
    """LayerNorm over the last axis in fp32, returned in ``x.dtype`` (reference: primitives.py:90-115)."""
    w = None if weight is None else weight.float()
    b = None if bias is None else bias.float()
    return F.layer_norm(x.float(), (x.shape[-1],), w, b, eps).to(x.dtype)


def swiglu(x):
    a, b = x.chunk(2, dim=-1)
    return F.silu(a) * b


def transition(x, ln_w, ln_b, w1, w2, eps: float = 1e-5):
    """``swiglu(LN(x) @ w1.T) @ w2.T`` (reference: primitives.py:248-251)."""
    h = F.linear(layer_norm(x, ln_w, ln_b, eps), w1)
    return F.linear(swiglu(h), w2)


def dropout_add(residual, x, p: float, training: bool, share_dim: int, mask=None):
    """``residual + dropout(x)`` with one Bernoulli draw shared along ``share_dim``.

    ``share_dim=-3`` shares the draw along rows, ``-2`` along columns
    (reference: triton/dropout_add.py:206-265). ``mask`` (already scaled by
    1/(1-p)) can be passed to make the result reproducible in tests.
    """
    if not training or p == 0.0:
        return residual + x
    if mask is None:
        shape = list(x.shape)
        shape[share_dim] = 1
        mask = F.dropout(x.new_ones(shape), p=p, training=True)
    return residual + x * mask


def pair_bias_attention(q, k, v, bias, key_mask, scale: float, fp32_qk: bool = False):
    """Softmax attention with an additive bias shared over rows.

    Args:
        q, k, v: ``[B, R, H, N, D]``.
        bias: ``[B, H, N, N]`` indexed (query token, key token), or ``None``.
        key_mask: ``[B, R, N]`` with 1 = attend, 0 = masked, or ``None``.
        scale: multiplies ``q·k``.
        fp32_qk: form ``q·k`` from fp32 copies of q and k (the diffusion
            transformer's contract, reference diffusion.py:536-540).

    Returns ``[B, R, H, N, D]`` in ``v.dtype``. The logits and softmax are
    fp32 (reference: attention.py:143-165).
    """
    if fp32_qk:
        logits = torch.matmul(q.float(), k.float().transpose(-2, -1)) * scale
    else:
        logits = torch.matmul(q, k.transpose(-2, -1)).float() * scale
    if bias is not None:
        logits = logits + bias.float().unsqueeze(1)
    if key_mask is not None:
        logits = logits + MASK_NEG * (key_mask.float() - 1.0)[:, :, None, None, :]
    w = torch.softmax(logits, dim=-1).to(v.dtype)
    return torch.matmul(w, v)


def window_attention(q, k, v, bias, scale: float):
    """Attention inside atom windows: ``softmax(q k^T * scale + bias) v``.

    ``q``: ``[..., H, Q, D]``; ``k``, ``v``: ``[..., H, K, D]``; ``bias``
    broadcastable to ``[..., H, Q, K]`` and already holding the key mask.
    Softmax in fp32 (reference: atom_cross_attn.py:764-769).
    """
    logits = torch.matmul(q, k.transpose(-2, -1)).float() * scale + bias.float()
    return torch.matmul(torch.softmax(logits, dim=-1).to(v.dtype), v)


def triangle_contract(a, b, outgoing: bool):
    """``out[i,j,c] = sum_k a[i,k,c] b[j,k,c]`` (outgoing) or ``sum_k a[k,j,c] b[k,i,c]`` (incoming).

    ``a``, ``b``: ``[B, N, N, C]``; reference: ops.py:58-92.
    """
    ac, bc = a.permute(0, 3, 1, 2), b.permute(0, 3, 1, 2)
    if outgoing:
        out = torch.matmul(ac, bc.transpose(-1, -2))
    else:
        out = torch.matmul(bc.transpose(-1, -2), ac)
    return out.permute(0, 2, 3, 1)


def gated_dual_linear(x, w_gate, w_proj, mask=None):
    """``sigmoid(x @ w_gate.T) * (x @ w_proj.T) * mask[..., None]``."""
    out = torch.sigmoid(F.linear(x, w_gate)) * F.linear(x, w_proj)
    return out if mask is None else out * mask.unsqueeze(-1).to(out.dtype)


def outer_product_mean(a, b, out_w, out_b, mask, eps: float = 1e-3, mask_i=None, mask_j=None):
    """``(sum_s a[s,i,:] (x) b[s,j,:]) . out_w + out_b``, divided by the count of valid rows.

    ``a``: ``[B, S, Ni, E]`` and ``b``: ``[B, S, Nj, E]`` already masked;
    ``out_w``: ``[E, E, C]``; ``mask``: ``[B, S, N]`` used for both sides unless
    ``mask_i`` / ``mask_j`` give the two sides of a tile (reference: ops.py:705-785).
    """
    mi = (mask if mask_i is None else mask_i).float()
    mj = (mask if mask_j is None else mask_j).float()
    ab = torch.einsum("bsie,bsjf->bijef", a, b)
    act = torch.einsum("bijef,efc->bijc", ab, out_w.to(ab.dtype)) + out_b.to(ab.dtype)
    norm = torch.einsum("bsi,bsj->bij", mi, mj)
    return act / (eps + norm.unsqueeze(-1)).to(act.dtype)


def msa_weighted_average(w, v):
    """``out[b,s,q,h,:] = sum_k w[b,h,q,k] v[b,s,k,h,:]`` (reference: attention.py:314)."""
    return torch.einsum("bhqk,bskhc->bsqhc", w, v)


def adamw_ema_step(
    params, grads, exp_avgs, exp_avg_sqs, shadows, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale, ema_decay
):
    """One AdamW step on lists of fp32 tensors, then ``shadow.lerp_(param, 1 - ema_decay)``.

    ``grads`` are multiplied by ``grad_scale`` first (the clip coefficient
    times 1/world). Matches ``torch.optim.AdamW`` (decoupled decay) followed by
    the reference's EMA update (training/ema.py:77-90).
    """
    bc1 = 1.0 - beta1**step
    bc2 = 1.0 - beta2**step
    for i, p in enumerate(params):
        g = grads[i].float() * grad_scale
        if weight_decay != 0.0:
            p.mul_(1.0 - lr * weight_decay)
        exp_avgs[i].lerp_(g, 1.0 - beta1)
        exp_avg_sqs[i].mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        denom = (exp_avg_sqs[i].sqrt() / (bc2**0.5)).add_(eps)
        p.addcdiv_(exp_avgs[i], denom, value=-lr / bc1)
        if shadows is not None and shadows[i] is not None:
            shadows[i].lerp_(p, 1.0 - ema_decay)
