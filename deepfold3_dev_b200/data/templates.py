"""Template features from aligned template chains (reference: data/feature/featurizer.py:420-560).

Inputs are template hits whose coordinates are already available as arrays (a chain's residue names and
per-residue atom coordinates in ``const.RESIDUE_ATOMS`` order); reading them out of mmCIF files is the
preparation step that needs gemmi. Features, per template ``t`` and query token ``i``:
``template_aatype``, ``template_pseudo_beta`` (+ mask: CB, or CA for glycine), ``template_backbone_frame`` (+ mask:
rows e1, e2, e3 from N, CA, C), ``template_ca``, ``template_mask``.
"""

from __future__ import annotations

import dataclasses

import numpy as np
import torch

from . import const


@dataclasses.dataclass
class TemplateChain:
    res_names: list  # three-letter names, one per template residue
    coords: np.ndarray  # [L, 24, 3] atoms in const.RESIDUE_ATOMS order
    atom_mask: np.ndarray  # [L, 24] bool
    query_to_hit: dict  # 0-based query residue -> 0-based template residue


def _frames(n, ca, c):
    e1 = c - ca
    e1 = e1 / np.linalg.norm(e1, axis=-1, keepdims=True).clip(1e-8)
    u = n - ca
    e2 = u - e1 * (u * e1).sum(-1, keepdims=True)
    e2 = e2 / np.linalg.norm(e2, axis=-1, keepdims=True).clip(1e-8)
    return np.stack([e1, e2, np.cross(e1, e2)], axis=-2)


def template_features(query_len: int, templates: list[TemplateChain], max_templates: int = 4, token_offset: int = 0,
                      num_tokens: int | None = None) -> dict:  # fmt: skip
    """Features of up to ``max_templates`` templates for a chain occupying tokens ``[offset, offset + query_len)``."""
    n = num_tokens or query_len
    T = max_templates
    out = {
        "template_aatype": torch.full((T, n), const.RES_TYPE_ORDER["-"], dtype=torch.long),
        "template_pseudo_beta": torch.zeros(T, n, 3), "template_pseudo_beta_mask": torch.zeros(T, n),
        "template_backbone_frame": torch.eye(3).expand(T, n, 3, 3).clone(), "template_backbone_mask": torch.zeros(T, n),
        "template_ca": torch.zeros(T, n, 3), "template_mask": torch.zeros(T),
    }  # fmt: skip
    for t, tpl in enumerate(templates[:T]):
        out["template_mask"][t] = 1.0
        for q, h in tpl.query_to_hit.items():
            if not (0 <= q < query_len and 0 <= h < len(tpl.res_names)):
                continue
            i = token_offset + q
            name = tpl.res_names[h]
            out["template_aatype"][t, i] = const.RES_TYPE_ORDER.get(name, const.RES_TYPE_ORDER["UNK"])
            atoms = const.RESIDUE_ATOMS.get(name, const.RESIDUE_ATOMS["UNK"])
            xyz, ok = tpl.coords[h], tpl.atom_mask[h]
            idx = {a: k for k, a in enumerate(atoms)}
            if all(a in idx and ok[idx[a]] for a in ("N", "CA", "C")):
                fr = _frames(xyz[idx["N"]], xyz[idx["CA"]], xyz[idx["C"]])
                out["template_backbone_frame"][t, i] = torch.as_tensor(fr, dtype=torch.float32)
                out["template_backbone_mask"][t, i] = 1.0
                out["template_ca"][t, i] = torch.as_tensor(xyz[idx["CA"]], dtype=torch.float32)
            pb = "CB" if ("CB" in idx and ok[idx["CB"]]) else "CA"
            if pb in idx and ok[idx[pb]]:
                out["template_pseudo_beta"][t, i] = torch.as_tensor(xyz[idx[pb]], dtype=torch.float32)
                out["template_pseudo_beta_mask"][t, i] = 1.0
    return out
