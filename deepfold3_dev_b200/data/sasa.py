"""Solvent-accessible surface (Shrake-Rupley) and the per-token burial targets derived from it.

Reference: data/sasa.py:108-382 (golden-spiral sphere, probe 1.4 A, per-token dSASA / contact-count targets against
each partner chain). The surface routine here walks atoms through fixed-radius neighbour lists: for one atom the sphere
points are tested against its neighbours only, so cost is linear in the number of atoms.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
from scipy.spatial import cKDTree

PROBE = 1.4
N_POINTS = 96
_VDW = {1: 1.10, 6: 1.70, 7: 1.55, 8: 1.52, 9: 1.47, 12: 1.73, 15: 1.80, 16: 1.80, 17: 1.75, 20: 2.31, 26: 2.04, 30: 1.39,
        34: 1.90, 35: 1.85, 53: 1.98}  # fmt: skip
VDW_BY_Z = np.full(128, 1.70)
for _z, _r in _VDW.items():
    VDW_BY_Z[_z] = _r


def sphere_points(n: int) -> np.ndarray:
    """Golden-spiral points on the unit sphere, [n, 3]."""
    k = np.arange(n) + 0.5
    polar = np.arccos(1.0 - 2.0 * k / n)
    azim = np.pi * (1.0 + 5.0**0.5) * k
    return np.stack([np.cos(azim) * np.sin(polar), np.sin(azim) * np.sin(polar), np.cos(polar)], axis=1)


def atom_sasa(xyz: np.ndarray, radii: np.ndarray, probe: float = PROBE, n_points: int = N_POINTS,
              query: np.ndarray | None = None, occluders: np.ndarray | None = None) -> np.ndarray:  # fmt: skip
    """Accessible area (A^2) of the ``query`` atoms (default all) with ``occluders`` (bool mask, default all) present."""
    xyz = np.asarray(xyz, dtype=np.float64)
    ext = np.asarray(radii, dtype=np.float64) + probe
    query = np.arange(len(xyz)) if query is None else np.asarray(query)
    out = np.zeros(len(query))
    if not len(xyz) or not len(query):
        return out
    occ = np.arange(len(xyz)) if occluders is None else np.nonzero(occluders)[0]
    tree = cKDTree(xyz[occ])
    unit = sphere_points(n_points)
    reach = float(ext[occ].max()) if len(occ) else 0.0
    lists = tree.query_ball_point(xyz[query], ext[query] + reach)
    for k, (i, nb) in enumerate(zip(query, lists)):
        nb = occ[np.asarray(nb, dtype=np.int64)]
        nb = nb[nb != i]
        area = 4.0 * np.pi * ext[i] ** 2
        if not len(nb):
            out[k] = area
            continue
        close = nb[np.linalg.norm(xyz[nb] - xyz[i], axis=1) < ext[nb] + ext[i]]
        if not len(close):
            out[k] = area
            continue
        pts = xyz[i] + ext[i] * unit  # [P, 3]
        d2 = ((pts[:, None, :] - xyz[close][None]) ** 2).sum(-1)
        out[k] = area * float((d2 >= ext[close][None] ** 2).all(1).mean())
    return out


@dataclass
class BurialTargets:
    """Token-level targets: ``dsasa[n, c]`` is the area token ``n`` loses when partner chain ``partner_asym[c]`` is added
    to its own chain; ``n_contact`` counts its heavy-atom contacts with that chain; ``loss_mask`` marks defined pairs."""

    dsasa: np.ndarray
    n_contact: np.ndarray
    loss_mask: np.ndarray
    partner_asym: np.ndarray
    sasa_chain: np.ndarray
    own_asym: np.ndarray

    def buried_area(self) -> dict[tuple[int, int], float]:
        """Buried surface per chain pair (half the summed loss of both sides)."""
        out: dict[tuple[int, int], float] = {}
        for c, pc in enumerate(self.partner_asym):
            for a in np.unique(self.own_asym[self.loss_mask[:, c]]):
                key = (int(min(a, pc)), int(max(a, pc)))
                sel = self.loss_mask[:, c] & (self.own_asym == a)
                out[key] = out.get(key, 0.0) + float(self.dsasa[sel, c].sum()) / 2.0
        return out


def burial_targets(atom_pos, atom_mask, elements, asym_id, seq_mask, partner_asym=None, probe: float = PROBE,
                   n_points: int = N_POINTS, shell: float = 8.0, contact_dist: float = 4.5) -> BurialTargets:  # fmt: skip
    """Dense token-atom layout in (``atom_pos`` [N, M, 3], ``atom_mask`` [N, M], ``elements`` [N, M]) -> targets.

    Only atoms within ``shell`` of a partner chain can lose area when that chain is added, so the pairwise surface is
    evaluated for those atoms only.
    """
    atom_mask = np.asarray(atom_mask, bool) & np.asarray(seq_mask, bool)[:, None]
    tok, slot = np.nonzero(atom_mask)
    xyz = np.asarray(atom_pos, np.float64)[tok, slot]
    rad = VDW_BY_Z[np.clip(np.asarray(elements)[tok, slot].astype(np.int64), 0, 127)]
    asym_id = np.asarray(asym_id)
    chain = asym_id[tok]
    n_tok = atom_mask.shape[0]
    partner_asym = np.unique(chain) if partner_asym is None else np.asarray(partner_asym)
    K = len(partner_asym)
    out = BurialTargets(np.zeros((n_tok, K), np.float32), np.zeros((n_tok, K), np.float32), np.zeros((n_tok, K), bool),
                        partner_asym.astype(np.int64), np.zeros(n_tok, np.float32), asym_id.copy())  # fmt: skip
    if not len(xyz):
        return out
    alone = np.zeros(len(xyz))
    for a in np.unique(chain):
        idx = np.nonzero(chain == a)[0]
        alone[idx] = atom_sasa(xyz, rad, probe, n_points, query=idx, occluders=chain == a)
    np.add.at(out.sasa_chain, tok, alone.astype(np.float32))
    trees = {int(a): cKDTree(xyz[chain == a]) for a in np.unique(chain)}
    for c, pc in enumerate(partner_asym):
        if int(pc) not in trees:
            continue
        for a in np.unique(chain):
            if a == pc:
                continue
            idx = np.nonzero(chain == a)[0]
            out.loss_mask[np.unique(tok[idx]), c] = True
            dist, _ = trees[int(pc)].query(xyz[idx], distance_upper_bound=shell)
            near = idx[np.isfinite(dist)]
            if not len(near):
                continue
            both = atom_sasa(xyz, rad, probe, n_points, query=near, occluders=(chain == a) | (chain == pc))
            np.add.at(out.dsasa[:, c], tok[near], np.maximum(alone[near] - both, 0.0).astype(np.float32))
            counts = trees[int(pc)].query_ball_point(xyz[near], contact_dist, return_length=True)
            np.add.at(out.n_contact[:, c], tok[near], counts.astype(np.float32))
    return out
