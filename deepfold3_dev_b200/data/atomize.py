"""Stochastic atomisation of standard residues in training (reference: data/tokenize/atomize.py:109-319).

With probability ``p_example`` an example gets some of its standard polymer residues re-tokenised as one token per
heavy atom (the representation ligands and modified residues always use), so the model also sees standard chemistry
through the atom-token path. Works on the feature dict: the chosen residue tokens are replaced by per-atom tokens
that share the residue index, chain ids and reference conformer (``ref_space_uid``), MSA columns and template rows
are repeated for them, and frames are dropped for atom tokens.
"""

from __future__ import annotations

import torch

from . import const
from .cropper import select_tokens


def select_residues_to_atomize(feats: dict, gen: torch.Generator, fraction: float = 0.05, max_residues: int = 8) -> torch.Tensor:
    polymer = (feats["mol_type"] != const.MOL_NONPOLYMER) & feats["seq_mask"].bool() & (feats["ref_mask"].sum(-1) > 1)
    idx = torch.nonzero(polymer).flatten()
    if len(idx) == 0:
        return idx
    k = min(max_residues, max(1, int(round(fraction * len(idx)))))
    return idx[torch.randperm(len(idx), generator=gen)[:k]].sort().values


def atomize_tokens(feats: dict, residues: torch.Tensor) -> dict:
    """Replace every token in ``residues`` by one token per heavy atom."""
    if len(residues) == 0:
        return feats
    n = int(feats["res_type"].shape[0])
    chosen = set(residues.tolist())
    order, atom_slot = [], []
    for i in range(n):
        if i in chosen:
            k = int(feats["ref_mask"][i].sum())
            order += [i] * k
            atom_slot += list(range(k))
        else:
            order.append(i)
            atom_slot.append(-1)
    order_t, slot_t = torch.tensor(order), torch.tensor(atom_slot)
    out = select_tokens(feats, order_t)  # repeats rows / columns of every token axis
    is_atom = slot_t >= 0
    m = len(order)
    ar = torch.arange(m)
    for key in ("ref_pos", "ref_mask", "ref_element", "ref_charge", "ref_atom_name_chars", "atom_gt_positions", "atom_gt_mask"):
        if key not in out:
            continue
        src = out[key]
        new = torch.zeros_like(src)
        new[~is_atom] = src[~is_atom]
        new[ar[is_atom], 0] = src[ar[is_atom], slot_t[is_atom]]  # the token's single atom moves to slot 0
        out[key] = new
    out["token_to_rep_atom"] = torch.where(is_atom, 0, out["token_to_rep_atom"])
    out["token_to_center_atom"] = torch.where(is_atom, 0, out["token_to_center_atom"])
    out["frames_mask"] = out["frames_mask"] & ~is_atom
    out["res_type"] = out["res_type"].clone()  # residue identity is kept (an atomised ALA is still ALA), as in the reference
    out["is_atomized"] = is_atom
    return out


def maybe_atomize(feats: dict, gen: torch.Generator, p_example: float = 0.1, fraction: float = 0.05, max_residues: int = 8) -> dict:
    if p_example <= 0 or float(torch.rand((), generator=gen)) >= p_example:
        return feats
    return atomize_tokens(feats, select_residues_to_atomize(feats, gen, fraction, max_residues))


def atomize_stored_features(feats: dict, gen: torch.Generator, prob: float, max_residues: int = 0) -> dict:
    """The recipe's ``atomize_prob`` / ``atomize_max_residues`` for examples stored as feature files, which cannot be
    tokenised again: every standard polymer residue token is picked with probability ``prob``, at most
    ``max_residues`` (0: no cap). Examples built from structures are atomised at tokenisation instead
    (``featurize.tokenize_structure``), where the residue's chemical bonds are also known; here the bond matrix keeps
    the rows of the residue token it was copied from."""
    if prob <= 0:
        return feats
    polymer = (feats["mol_type"] != const.MOL_NONPOLYMER) & feats["seq_mask"].bool() & (feats["ref_mask"].sum(-1) > 1)
    idx = torch.nonzero(polymer).flatten()
    idx = idx[torch.rand(len(idx), generator=gen) < prob]
    if max_residues > 0 and len(idx) > max_residues:
        idx = idx[torch.randperm(len(idx), generator=gen)[:max_residues]].sort().values
    return atomize_tokens(feats, idx)
