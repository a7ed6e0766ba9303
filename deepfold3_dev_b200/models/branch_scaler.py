"""Function applied to each residual-branch output before its block multiplier.

``identity`` keeps the AF3 behaviour; ``rmsnorm`` rescales every branch to unit
RMS per token (reference: model/branch_scaler.py:31-65).
"""

from __future__ import annotations

import torch.nn as nn

from .primitives import rms_normalize


class IdentityScaler(nn.Module):
    def forward(self, x):
        return x


class RMSNormScaler(nn.Module):
    def forward(self, x):
        return rms_normalize(x)


def make_branch_scaler(kind: str) -> nn.Module:
    if kind == "identity":
        return IdentityScaler()
    if kind == "rmsnorm":
        return RMSNormScaler()
    raise ValueError(f"Unknown branch_scaler kind: {kind!r}")
