"""Superposition-based and superposition-free accuracy metrics on matched coordinate sets (numpy, CPU).

Reference: the accuracy scripts at the reference's repo root (``struct_accuracy.py``: lDDT / RMSD per target,
``gdt_ts.py``, ``usalign_tm.py`` which shells out to US-align, ``check_chirality.py``) and bench/ (DockQ through an
external tool). Here every metric is computed in-process: TM-score uses the sequence-dependent superposition search of
the TM-score program (seeded fragments, iterated re-superposition on residues under a distance cut-off), DockQ follows
its published definition (fnat, interface RMSD, ligand RMSD).
"""

from __future__ import annotations

import numpy as np
from scipy.spatial import cKDTree


def kabsch(mobile: np.ndarray, target: np.ndarray, weights: np.ndarray | None = None):
    """Rotation ``R`` and translation ``t`` minimising ``|| (mobile @ R.T + t) - target ||`` (weighted)."""
    w = np.ones(len(mobile)) if weights is None else np.asarray(weights, float)
    w = w / w.sum()
    cm, ct = (w[:, None] * mobile).sum(0), (w[:, None] * target).sum(0)
    h = (w[:, None] * (mobile - cm)).T @ (target - ct)
    u, _, vt = np.linalg.svd(h)
    d = np.sign(np.linalg.det(vt.T @ u.T))
    r = vt.T @ np.diag([1.0, 1.0, d]) @ u.T
    return r, ct - r @ cm


def superpose(mobile, target, weights=None):
    r, t = kabsch(mobile, target, weights)
    return mobile @ r.T + t


def rmsd(a: np.ndarray, b: np.ndarray, align: bool = True) -> float:
    a = superpose(a, b) if align else a
    return float(np.sqrt(((a - b) ** 2).sum(-1).mean()))


def lddt(pred: np.ndarray, true: np.ndarray, cutoff: float = 15.0, residue_of: np.ndarray | None = None,
         per_atom: bool = False, thresholds=(0.5, 1.0, 2.0, 4.0)):  # fmt: skip
    """Local distance difference test over all atom pairs closer than ``cutoff`` in ``true``.

    Pairs inside one residue are skipped when ``residue_of`` (residue index per atom) is given.
    """
    tree = cKDTree(true)
    pairs = tree.query_pairs(cutoff, output_type="ndarray")
    if residue_of is not None and len(pairs):
        pairs = pairs[residue_of[pairs[:, 0]] != residue_of[pairs[:, 1]]]
    if not len(pairs):
        return np.zeros(len(true)) if per_atom else 0.0
    dt = np.linalg.norm(true[pairs[:, 0]] - true[pairs[:, 1]], axis=1)
    dp = np.linalg.norm(pred[pairs[:, 0]] - pred[pairs[:, 1]], axis=1)
    kept = np.mean([(np.abs(dt - dp) < th) for th in thresholds], axis=0)
    if not per_atom:
        return float(kept.mean())
    total, count = np.zeros(len(true)), np.zeros(len(true))
    for col in (0, 1):
        np.add.at(total, pairs[:, col], kept)
        np.add.at(count, pairs[:, col], 1.0)
    return total / np.maximum(count, 1.0)


def _search_superposition(pred, true, score_fn, d_cut: float):
    """Best ``score_fn(distances)`` over superpositions grown from fragments (lengths L, L/2, L/4, ... >= 4)."""
    n = len(pred)
    best = 0.0
    size = n
    while size >= min(4, n):
        step = max(1, size // 2)
        for start in range(0, n - size + 1, step):
            idx = np.arange(start, start + size)
            for _ in range(20):
                moved = pred @ (rt := kabsch(pred[idx], true[idx]))[0].T + rt[1]
                d = np.linalg.norm(moved - true, axis=1)
                best = max(best, score_fn(d))
                new = np.nonzero(d < d_cut)[0]
                if len(new) < 3 or np.array_equal(new, idx):
                    break
                idx = new
        if size == min(4, n):
            break
        size = max(min(4, n), size // 2)
    return best


def tm_score(pred: np.ndarray, true: np.ndarray, l_norm: int | None = None) -> float:
    """TM-score of matched CA (or C1') traces, normalised by ``l_norm`` (default: length of ``true``)."""
    L = l_norm or len(true)
    d0 = max(0.5, 1.24 * (max(L, 19) - 15) ** (1.0 / 3.0) - 1.8)
    return _search_superposition(pred, true, lambda d: float((1.0 / (1.0 + (d / d0) ** 2)).sum() / L), max(d0, 4.5))


def gdt_ts(pred: np.ndarray, true: np.ndarray) -> float:
    """Mean over 1, 2, 4, 8 A of the largest fraction of residues that can be superposed under the cut-off."""
    return float(np.mean([_search_superposition(pred, true, lambda d, c=c: float((d <= c).mean()), c) for c in (1.0, 2.0, 4.0, 8.0)]))


def dockq(pred_rec, pred_lig, true_rec, true_lig, rec_bb=None, lig_bb=None) -> dict:
    """DockQ of a receptor / ligand chain pair from matched atoms (``[n, 3]`` each; ``*_bb`` mark backbone atoms).

    fnat: fraction of native atom contacts (< 5 A) kept; iRMSD: backbone RMSD of the native interface (atoms within
    10 A of the partner) after superposing it; LRMSD: ligand backbone RMSD after superposing the receptor.
    """
    rec_bb = np.ones(len(true_rec), bool) if rec_bb is None else rec_bb
    lig_bb = np.ones(len(true_lig), bool) if lig_bb is None else lig_bb
    native = cKDTree(true_rec).query_ball_tree(cKDTree(true_lig), 5.0)
    pairs = np.array([(i, j) for i, js in enumerate(native) for j in js], dtype=np.int64).reshape(-1, 2)
    if not len(pairs):
        return {"fnat": 0.0, "irmsd": float("nan"), "lrmsd": float("nan"), "dockq": 0.0}
    kept = np.linalg.norm(pred_rec[pairs[:, 0]] - pred_lig[pairs[:, 1]], axis=1) < 5.0
    fnat = float(kept.mean())
    near_r = np.isfinite(cKDTree(true_lig).query(true_rec, distance_upper_bound=10.0)[0]) & rec_bb
    near_l = np.isfinite(cKDTree(true_rec).query(true_lig, distance_upper_bound=10.0)[0]) & lig_bb
    it, ip = np.concatenate([true_rec[near_r], true_lig[near_l]]), np.concatenate([pred_rec[near_r], pred_lig[near_l]])
    irmsd = rmsd(ip, it)
    r, t = kabsch(pred_rec[rec_bb], true_rec[rec_bb])
    lrmsd = float(np.sqrt((((pred_lig[lig_bb] @ r.T + t) - true_lig[lig_bb]) ** 2).sum(-1).mean()))
    score = (fnat + 1.0 / (1.0 + (irmsd / 1.5) ** 2) + 1.0 / (1.0 + (lrmsd / 8.5) ** 2)) / 3.0
    return {"fnat": fnat, "irmsd": irmsd, "lrmsd": lrmsd, "dockq": float(score)}


def chirality_violations(xyz: np.ndarray, centers: np.ndarray, reference_xyz: np.ndarray) -> float:
    """Fraction of chiral centres whose signed volume differs in sign from the reference.

    ``centers`` is ``[k, 4]`` atom indices: the centre and three neighbours in a fixed order.
    """
    if not len(centers):
        return 0.0

    def vol(p):
        a, b, c = (p[centers[:, k]] - p[centers[:, 0]] for k in (1, 2, 3))
        return np.einsum("ij,ij->i", a, np.cross(b, c))

    return float((np.sign(vol(xyz)) != np.sign(vol(reference_xyz))).mean())
