"""Token crops of a featurised example (reference: data/crop/cropper.py:86-772).

Three strategies with weights 0.2 / 0.4 / 0.4: contiguous (per-chain contiguous segments, AF-Multimer
algorithm 1), spatial (the ``max_tokens`` tokens nearest to a reference token) and spatial-interface
(the reference token is drawn among tokens within 15 Angstrom of another chain). Both a token and an
atom budget apply. Cropping works on the feature dict: every token axis is re-indexed, MSA columns and
template rows follow.
"""

from __future__ import annotations

import torch

from ..models.bucket import _token_axes

CROP_WEIGHTS = {"contiguous": 0.2, "spatial": 0.4, "spatial_interface": 0.4}
INTERFACE_DISTANCE = 15.0


def _center_coords(feats):
    n = feats["res_type"].shape[0]
    pos = feats["atom_gt_positions"] if "atom_gt_positions" in feats else feats["ref_pos"]
    idx = feats["token_to_center_atom"].view(n, 1, 1).expand(n, 1, 3)
    ok = feats["atom_gt_mask"].gather(1, feats["token_to_center_atom"].view(n, 1)).squeeze(1) if "atom_gt_mask" in feats else torch.ones(n, dtype=torch.bool)
    return pos.gather(1, idx).squeeze(1), ok.bool()


def contiguous_crop(asym_id: torch.Tensor, max_tokens: int, gen: torch.Generator) -> torch.Tensor:
    """Indices kept by the contiguous multi-chain crop (chains visited in random order)."""
    chains = torch.unique(asym_id)
    chains = chains[torch.randperm(len(chains), generator=gen)]
    remaining = int(sum(int((asym_id == c).sum()) for c in chains))
    budget, keep = max_tokens, []
    for c in chains:
        idx = torch.nonzero(asym_id == c).flatten()
        n = len(idx)
        remaining -= n
        hi = min(budget, n)
        lo = min(n, max(0, budget - remaining))
        size = int(torch.randint(lo, hi + 1, (1,), generator=gen)) if hi >= lo else hi
        budget -= size
        if size > 0:
            start = int(torch.randint(0, n - size + 1, (1,), generator=gen))
            keep.append(idx[start : start + size])
        if budget <= 0:
            break
    return torch.sort(torch.cat(keep)).values if keep else torch.arange(min(max_tokens, len(asym_id)))


def spatial_crop(coords, valid, asym_id, max_tokens: int, gen: torch.Generator, interface: bool) -> torch.Tensor:
    cand = valid.clone()
    if interface:
        d = torch.cdist(coords, coords)
        other = asym_id[:, None] != asym_id[None, :]
        near = ((d < INTERFACE_DISTANCE) & other & valid[None, :]).any(-1) & valid
        if bool(near.any()):
            cand = near
    pool = torch.nonzero(cand).flatten()
    if len(pool) == 0:
        pool = torch.arange(len(asym_id))
    ref = pool[int(torch.randint(0, len(pool), (1,), generator=gen))]
    dist = (coords - coords[ref]).norm(dim=-1) + (~valid).float() * 1e6
    dist = dist + torch.arange(len(dist)) * 1e-3  # deterministic tie-break
    return torch.sort(torch.topk(dist, min(max_tokens, len(dist)), largest=False).indices).values


def apply_atom_budget(keep: torch.Tensor, ref_mask: torch.Tensor, max_atoms: int) -> torch.Tensor:
    if max_atoms <= 0:
        return keep
    counts = ref_mask[keep].sum(-1).cumsum(0)
    return keep[counts <= max_atoms]


def select_tokens(feats: dict, keep: torch.Tensor) -> dict:
    """Re-index every token axis of ``feats`` to the kept tokens."""
    n = int(feats["res_type"].shape[0])
    out = {}
    for k, v in feats.items():
        if not isinstance(v, torch.Tensor) or v.dim() == 0:
            out[k] = v
            continue
        t = v
        for axis in _token_axes(k, v, n):
            t = t.index_select(axis, keep)
        out[k] = t
    m = len(keep)
    out["token_index"] = torch.arange(m)
    if "frame_token_index" in out:  # frames point at tokens: keep only frames whose tokens survived, renumbered
        new_of_old = torch.full((n,), -1, dtype=torch.long)
        new_of_old[keep] = torch.arange(m)
        fti = new_of_old[feats["frame_token_index"].index_select(0, keep)]
        alive = (fti >= 0).all(-1)
        out["frame_token_index"] = torch.where(fti >= 0, fti, torch.arange(m).unsqueeze(-1).expand(m, 3))
        out["frames_mask"] = out["frames_mask"] & alive
    return out


def crop(feats: dict, max_tokens: int, max_atoms: int = 0, gen: torch.Generator | None = None, weights: dict | None = None,
         strategy: str | None = None, return_keep: bool = False):  # fmt: skip
    """Crop to the budgets; returns the cropped features and the strategy used (with ``return_keep`` also the sorted
    indices of the tokens kept, ``None`` when nothing was cut)."""
    out = _crop(feats, max_tokens, max_atoms, gen, weights, strategy)
    return out if return_keep else out[:2]


def _crop(feats, max_tokens, max_atoms, gen, weights, strategy):
    gen = gen or torch.Generator().manual_seed(int(torch.randint(0, 2**31 - 1, (1,))))
    n = int(feats["res_type"].shape[0])
    w = weights or CROP_WEIGHTS
    if strategy is None:
        names = list(w)
        strategy = names[int(torch.multinomial(torch.tensor([float(w[k]) for k in names]), 1, generator=gen))]
    if n <= max_tokens and (max_atoms <= 0 or int(feats["ref_mask"].sum()) <= max_atoms):
        return feats, "none", None
    if strategy == "contiguous":
        keep = contiguous_crop(feats["asym_id"], max_tokens, gen)
    else:
        coords, valid = _center_coords(feats)
        keep = spatial_crop(coords.float(), valid, feats["asym_id"], max_tokens, gen, strategy == "spatial_interface")
    keep = apply_atom_budget(keep, feats["ref_mask"], max_atoms)
    return select_tokens(feats, keep), strategy, keep
