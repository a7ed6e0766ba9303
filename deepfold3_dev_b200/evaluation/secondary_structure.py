"""Secondary structure from C-alpha traces, and how well a prediction recovers it.

The reference follows secondary-structure learning over training with DSSP on full-atom models (scripts/dssp_f1.py,
scripts/ss_learning.py: per-class F1 against the experimental structure, and for every true helix the longest run of
predicted helix inside it). DSSP needs backbone hydrogen-bond geometry and an external program; the three-state
assignment here needs only consecutive C-alpha positions, so it also works on early checkpoints whose side chains and
carbonyls are still meaningless, and in-process on every sample of a sweep.
"""

from __future__ import annotations

import numpy as np

STATES = ("H", "E", "C")


def assign_ss(ca: np.ndarray) -> np.ndarray:
    """Three-state string array ``[L]`` (``H`` helix, ``E`` strand, ``C`` other) from C-alpha positions ``[L, 3]`` of
    consecutive residues. A five-residue window is helical when its i..i+2, i..i+3 and i..i+4 distances are those of
    an alpha helix (5.5, 5.3, 6.4 A within 0.6) and extended when they are 6.4, 9.8, 12.4 A (within 1.0 / 1.4 / 1.8);
    every residue of a matching window takes the state (helix wins where both claim a residue); runs shorter than three
    residues fall back to ``C``."""
    n = len(ca)
    out = np.full(n, "C", dtype="<U1")
    if n < 5:
        return out
    d = lambda k: np.linalg.norm(ca[k:] - ca[:-k], axis=-1)[: n - 4]  # noqa: E731
    d2, d3, d4 = d(2), d(3), d(4)
    helix = (abs(d2 - 5.5) < 0.6) & (abs(d3 - 5.3) < 0.6) & (abs(d4 - 6.4) < 0.6)
    strand = (abs(d2 - 6.4) < 1.0) & (abs(d3 - 9.8) < 1.4) & (abs(d4 - 12.4) < 1.8)
    for flags, state in ((strand, "E"), (helix, "H")):
        for i in np.nonzero(flags)[0]:
            out[i : i + 5] = state
    for state in ("H", "E"):  # drop runs too short to be an element
        for a, b in runs(out, state):
            if b - a < 3:
                out[a:b] = "C"
    return out


def runs(ss: np.ndarray, state: str) -> list[tuple[int, int]]:
    """Half-open index ranges of the maximal runs of ``state``."""
    hit = np.concatenate([[False], ss == state, [False]])
    edges = np.nonzero(hit[1:] != hit[:-1])[0]
    return list(zip(edges[0::2].tolist(), edges[1::2].tolist()))


def ss_agreement(pred_ca: np.ndarray, true_ca: np.ndarray) -> dict:
    """Per-state F1 and three-state accuracy of the prediction's assignment against the experimental one (same
    residues, same order), plus helix recovery: for every true helix, the longest run of predicted helix inside it
    divided by its length (helices tend to be recovered whole or not at all, so the distribution is bimodal)."""
    p, t = assign_ss(np.asarray(pred_ca, float)), assign_ss(np.asarray(true_ca, float))
    if len(p) != len(t):
        raise ValueError("ss_agreement needs traces of the same residues")
    out = {"q3": float((p == t).mean()) if len(t) else float("nan")}
    for s, name in zip(STATES, ("helix", "strand", "coil")):
        tp = int(((p == s) & (t == s)).sum())
        fp, fn = int(((p == s) & (t != s)).sum()), int(((p != s) & (t == s)).sum())
        out[f"f1_{name}"] = 2 * tp / (2 * tp + fp + fn) if (2 * tp + fp + fn) else float("nan")
    rec = []
    for a, b in runs(t, "H"):
        inside = runs(p[a:b], "H")
        rec.append(max((y - x for x, y in inside), default=0) / (b - a))
    out["helix_recovery"] = rec
    out["helix_recovery_mean"] = float(np.mean(rec)) if rec else float("nan")
    return out
