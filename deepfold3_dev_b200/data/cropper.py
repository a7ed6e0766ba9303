"""Token crops of a featurised example (reference: data/crop/cropper.py:86-772).

Three strategies with weights 0.2 / 0.4 / 0.4, drawn independently of the sampler's anchor (AF3 SI 2.7):

* contiguous: AF-Multimer algorithm 1: the chains are visited in random order and each contributes one contiguous
  segment whose length is drawn so that the token budget can still be met;
* spatial: the tokens nearest to a seed token, by the distance between token centre atoms;
* spatial-interface: the same with the seed drawn among tokens within 15 Angstrom of a token of another chain.

Only tokens whose centre atom is resolved are candidates of the two spatial strategies, so an unresolved stretch never
fills a crop. The sampler's anchor (the weighted chain or interface that made this example be drawn) biases the seed
only: a chain anchor restricts the seed pool to that chain, an interface anchor restricts interface seeds to tokens of
the two chains that touch the other one. Both a token and an atom budget apply, in the order in which a strategy
collects tokens (by distance, or chain by chain), so the budget never removes the tokens nearest to the seed. A crop
must contain at least ``min_resolved`` resolved tokens (the rigid alignment inside the loss needs them); otherwise a
new crop is drawn, up to ``max_attempts`` times. Cropping works on the feature dict: every token axis is re-indexed,
MSA columns and template rows follow.
"""

from __future__ import annotations

import torch

from ..models.bucket import _token_axes

CROP_WEIGHTS = {"contiguous": 0.2, "spatial": 0.4, "spatial_interface": 0.4}
INTERFACE_DISTANCE = 15.0
MIN_RESOLVED = 4
MAX_ATTEMPTS = 8


def _center_coords(feats):
    """Centre-atom position per token and whether that atom is resolved (always true for features without a ground truth)."""
    n = feats["res_type"].shape[0]
    pos = feats["atom_gt_positions"] if "atom_gt_positions" in feats else feats["ref_pos"]
    idx = feats["token_to_center_atom"].view(n, 1, 1).expand(n, 1, 3)
    ok = feats["atom_gt_mask"].gather(1, feats["token_to_center_atom"].view(n, 1)).squeeze(1) if "atom_gt_mask" in feats else torch.ones(n, dtype=torch.bool)
    return pos.gather(1, idx).squeeze(1), ok.bool()


def _atoms_per_token(feats) -> torch.Tensor:
    return feats["ref_mask"].sum(-1).long()


def _within_budgets(order: torch.Tensor, atoms: torch.Tensor, max_tokens: int, max_atoms: int) -> torch.Tensor:
    """The longest prefix of ``order`` (token indices in collection order) that meets both budgets, sorted."""
    order = order[:max_tokens]
    if max_atoms > 0 and len(order):
        fits = atoms[order].cumsum(0) <= max_atoms
        # stop at the first token that would exceed the budget (no skipping ahead to smaller tokens)
        order = order[: int(fits.long().cumprod(0).sum())]
    return torch.sort(order).values


def contiguous_crop(asym_id: torch.Tensor, max_tokens: int, gen: torch.Generator, atoms: torch.Tensor | None = None,
                    max_atoms: int = 0) -> torch.Tensor:  # fmt: skip
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
    order = torch.cat(keep) if keep else torch.arange(min(max_tokens, len(asym_id)))
    if atoms is None:
        return torch.sort(order).values
    return _within_budgets(order, atoms, max_tokens, max_atoms)


def _seed_pool(pool: torch.Tensor, asym_id: torch.Tensor, anchor_chain: int | None) -> torch.Tensor:
    """Seed candidates: the pool's tokens of the anchor chain when there are any, else the whole pool."""
    if anchor_chain is not None:
        mine = pool[asym_id[pool] == anchor_chain]
        if len(mine):
            return mine
    return pool


def spatial_crop(coords, valid, asym_id, max_tokens: int, gen: torch.Generator, interface: bool, atoms: torch.Tensor | None = None,
                 max_atoms: int = 0, anchor=None) -> torch.Tensor:  # fmt: skip
    """Nearest-neighbour crop around a seed. ``valid``: tokens with a resolved centre atom (the only candidates, unless
    there are none). ``anchor``: ``("chain", a, _)`` or ``("interface", a, b)`` in ``asym_id`` numbering, or ``None``."""
    n = len(asym_id)
    pool = torch.nonzero(valid).flatten()
    if len(pool) == 0:
        pool = torch.arange(n)
    anchor_chain = int(anchor[1]) if anchor is not None else None
    seeds = None
    if interface and len(pool) >= 2:
        pc, pa = coords[pool], asym_id[pool]
        close = torch.cdist(pc, pc) < INTERFACE_DISTANCE
        if anchor is not None and anchor[0] == "interface":
            a, b = int(anchor[1]), int(anchor[2])
            touches = ((pa == a)[:, None] & (pa == b)[None, :] & close).any(-1) | ((pa == b)[:, None] & (pa == a)[None, :] & close).any(-1)
        else:
            touches = (close & (pa[:, None] != pa[None, :])).any(-1)
        if bool(touches.any()):
            seeds = pool[touches]
    if seeds is None:  # plain spatial crop, or no interface token of the wanted kind
        seeds = _seed_pool(pool, asym_id, anchor_chain)
    ref = seeds[int(torch.randint(0, len(seeds), (1,), generator=gen))]
    dist = (coords[pool] - coords[ref]).norm(dim=-1) + torch.arange(len(pool)) * 1e-6  # index breaks ties
    order = pool[torch.argsort(dist)]
    if atoms is None:
        return torch.sort(order[:max_tokens]).values
    return _within_budgets(order, atoms, max_tokens, max_atoms)


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
         strategy: str | None = None, return_keep: bool = False, anchor=None, min_resolved: int = MIN_RESOLVED,
         max_attempts: int = MAX_ATTEMPTS):  # fmt: skip
    """Crop to the budgets; returns the cropped features and the strategy used (with ``return_keep`` also the sorted
    indices of the tokens kept, ``None`` when nothing was cut). ``anchor``: the sampler's chain or interface in
    ``asym_id`` numbering (see the module text); ``strategy`` pins the strategy instead of drawing it."""
    out = _crop(feats, max_tokens, max_atoms, gen, weights, strategy, anchor, min_resolved, max_attempts)
    return out if return_keep else out[:2]


def _draw(w: dict, gen: torch.Generator) -> str:
    names = list(w)
    total = sum(float(w[k]) for k in names)
    if total <= 0:
        return "contiguous"
    return names[int(torch.multinomial(torch.tensor([float(w[k]) for k in names]), 1, generator=gen))]


def _crop(feats, max_tokens, max_atoms, gen, weights, strategy, anchor=None, min_resolved=MIN_RESOLVED, max_attempts=MAX_ATTEMPTS):
    gen = gen or torch.Generator().manual_seed(int(torch.randint(0, 2**31 - 1, (1,))))
    n = int(feats["res_type"].shape[0])
    w = weights or CROP_WEIGHTS
    drawn = strategy or _draw(w, gen)  # drawn even when nothing is cut, so the random stream does not depend on the size
    atoms = _atoms_per_token(feats)
    if n <= max_tokens and (max_atoms <= 0 or int(atoms.sum()) <= max_atoms):
        return feats, "none", None
    coords, resolved = _center_coords(feats)
    coords = coords.float()
    attempts = max_attempts if int(resolved.sum()) >= min_resolved else 1
    keep, used = None, drawn
    for attempt in range(max(1, attempts)):
        used = drawn if attempt == 0 else (strategy or _draw(w, gen))
        if used == "contiguous":
            keep = contiguous_crop(feats["asym_id"], max_tokens, gen, atoms, max_atoms)
        else:
            keep = spatial_crop(coords, resolved, feats["asym_id"], max_tokens, gen, used == "spatial_interface", atoms,
                                max_atoms, anchor)  # fmt: skip
        if int(resolved[keep].sum()) >= min_resolved:
            break
    return select_tokens(feats, keep), used, keep
