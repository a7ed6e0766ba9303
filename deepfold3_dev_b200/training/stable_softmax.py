"""Softmax, log-softmax and cross-entropy that keep the target gradient at large logit margins
(reference: training/stable_softmax.py:38-119, after Barron et al., "A Fix for Softmax and Cross-Entropy").

The usual max-shifted form has the denominator ``1 + exp(-m)`` with ``m`` the margin of the largest logit over the
log-sum-exp of the rest; once ``exp(-m)`` falls below the rounding step of 1.0 (m of about 5.5 in bf16, 16.6 in fp32)
the target gradient becomes exactly zero while the others stay positive. Here the leading slot never enters a sum with
1.0: its shifted logit is exactly 0, the log-sum-exp runs over the other slots only, and the two are recombined through
``softplus``, whose derivative ``sigmoid`` stays accurate down to exponent underflow.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def _others_lse(shifted: torch.Tensor, index: torch.Tensor, dim: int) -> torch.Tensor:
    """Log-sum-exp over every slot except ``index`` (kept dim); ``-inf`` when there is no other slot."""
    hidden = shifted.scatter(dim, index, float("-inf"))
    return torch.logsumexp(hidden, dim=dim, keepdim=True)


def log_softmax(z: torch.Tensor, dim: int = -1) -> torch.Tensor:
    top = z.argmax(dim=dim, keepdim=True)
    shifted = z - z.gather(dim, top)  # the leading slot is exactly 0
    return shifted - F.softplus(_others_lse(shifted, top, dim))


def softmax(z: torch.Tensor, dim: int = -1) -> torch.Tensor:
    return log_softmax(z, dim).exp()


def logit_margin(z: torch.Tensor, target: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """``z_target - logsumexp(z_others)`` per position (``target`` holds class indices, shape of ``z`` without ``dim``)."""
    t = target.unsqueeze(dim)
    zt = z.gather(dim, t)
    return (zt - _others_lse(z - zt.detach(), t, dim) - zt.detach()).squeeze(dim)


def cross_entropy(z: torch.Tensor, target: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Per-position ``-log p_target = softplus(-margin)``; gradient of the target logit is ``-sigmoid(-margin)``."""
    return F.softplus(-logit_margin(z, target, dim))
