"""Feature constructors: relative-position encoding and distance histograms.

Reference: model/embedders.py:13-101 (AF3 ``create_relative_encoding`` and the
39-bin squared-distance histogram used by templates and the confidence head).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

DGRAM_MIN_BIN = 3.25
DGRAM_MAX_BIN = 50.75
DGRAM_NUM_BINS = 39


def compute_rel_feat_dim(max_relative_idx: int = 32, max_relative_chain: int = 2) -> int:
    return 2 * (2 * max_relative_idx + 2) + 1 + (2 * max_relative_chain + 2)


def _clipped_offset(idx: torch.Tensor, same: torch.Tensor, span: int) -> torch.Tensor:
    """One-hot of ``clip(idx_i - idx_j + span, 0, 2 span)``, with bin ``2 span + 1`` where ``same`` is False."""
    d = (idx.unsqueeze(-1) - idx.unsqueeze(-2) + span).clamp(0, 2 * span)
    d = torch.where(same, d, torch.full_like(d, 2 * span + 1))
    return F.one_hot(d, 2 * span + 2).float()


def create_relative_encoding(
    token_index, residue_index, asym_id, entity_id, sym_id, max_relative_idx: int = 32, max_relative_chain: int = 2
) -> torch.Tensor:
    """``[..., N, N, 139]``: residue offset (66) | token offset (66) | same entity (1) | chain offset (6)."""
    same_chain = asym_id.unsqueeze(-1) == asym_id.unsqueeze(-2)
    same_entity = entity_id.unsqueeze(-1) == entity_id.unsqueeze(-2)
    same_residue = same_chain & (residue_index.unsqueeze(-1) == residue_index.unsqueeze(-2))
    return torch.cat(
        [
            _clipped_offset(residue_index, same_chain, max_relative_idx),
            _clipped_offset(token_index, same_residue, max_relative_idx),
            same_entity.float().unsqueeze(-1),
            _clipped_offset(sym_id, same_entity, max_relative_chain),
        ],
        dim=-1,
    )


def dgram_from_positions(positions, min_bin=DGRAM_MIN_BIN, max_bin=DGRAM_MAX_BIN, num_bins=DGRAM_NUM_BINS):
    """One-hot histogram ``[..., N, N, num_bins]`` of pairwise squared distances between bin edges."""
    lower = torch.linspace(min_bin, max_bin, num_bins, device=positions.device) ** 2
    upper = torch.cat([lower[1:], torch.full((1,), 1e8, device=positions.device, dtype=lower.dtype)])  # no host copy
    d2 = (positions.unsqueeze(-2) - positions.unsqueeze(-3)).pow(2).sum(-1, keepdim=True)
    return ((d2 > lower) & (d2 < upper)).float()
