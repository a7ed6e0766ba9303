"""Predicted mmCIF against an experimental mmCIF: chain matching, atom matching, metrics per target.

Chains are paired by identical sequence (greedy over the lowest CA RMSD after a global superposition when an entity has
several copies), atoms by name inside matched residues; only atoms resolved in the experimental structure count.
"""

from __future__ import annotations

import itertools

import numpy as np

from ..data import const
from ..data.parse.mmcif import parse_mmcif
from . import metrics


def _chain_table(st):
    out = []
    for c in st.chains:
        res = st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]
        out.append({"asym": int(c["asym_id"]), "mol": int(c["mol_type"]), "seq": tuple(r["name"] for r in res), "res": res})
    return out


def _restrict(chain: dict, keep: list[int]) -> dict:
    res = chain["res"][keep]
    return dict(chain, res=res, seq=tuple(r["name"] for r in res))


def _numbering_overlap(p: dict, t: dict, min_identity: float = 0.9):
    """Residue rows of ``p`` and ``t`` paired by the identical blocks of a sequence alignment, when those cover at least
    ``min_identity`` of the shorter chain (constructs that differ by tags, numbering or a few mutations)."""
    import difflib

    a, b = [r["name"] for r in p["res"]], [r["name"] for r in t["res"]]
    blocks = difflib.SequenceMatcher(None, a, b, autojunk=False).get_matching_blocks()
    kp = [i + k for i, _, n in blocks for k in range(n)]
    kt = [j + k for _, j, n in blocks for k in range(n)]
    if len(kp) < 4 or len(kp) / max(min(len(a), len(b)), 1) < min_identity:
        return None
    return kp, kt


def _trace(st, chain) -> tuple[np.ndarray, np.ndarray]:
    want = b"CA" if chain["mol"] == const.MOL_PROTEIN else b"C1'"
    pts, ok = np.zeros((len(chain["res"]), 3)), np.zeros(len(chain["res"]), bool)
    xyz = st.coords()
    for k, r in enumerate(chain["res"]):
        atoms = st.atoms[int(r["atom_idx"]) : int(r["atom_idx"]) + int(r["atom_num"])]
        hit = np.nonzero((atoms["name"] == want) & atoms["is_present"])[0]
        if chain["mol"] == const.MOL_NONPOLYMER:
            hit = np.nonzero(atoms["is_present"])[0][:1]
        if len(hit):
            pts[k], ok[k] = xyz[int(r["atom_idx"]) + hit[0]], True
    return pts, ok


def match_chains(pred, true) -> list[tuple[dict, dict]]:
    """Pairs ``(pred chain, true chain)`` with equal sequences; copies of an entity are assigned to minimise trace RMSD."""
    tp, tt = _chain_table(pred), _chain_table(true)
    groups: dict[tuple, tuple[list, list]] = {}
    for c in tp:
        groups.setdefault(c["seq"], ([], []))[0].append(c)
    for c in tt:
        if c["seq"] in groups:
            groups[c["seq"]][1].append(c)
    pairs = []
    # polymer chains without an identical partner: fall back to the overlap of their residue numbering
    used_t = {id(c) for _, ts in groups.values() for c in ts}
    for seq, (ps, ts) in list(groups.items()):
        if ts or not ps or ps[0]["mol"] == const.MOL_NONPOLYMER:
            continue
        for p in ps:
            best = None
            for t in tt:
                if id(t) in used_t or t["mol"] != p["mol"]:
                    continue
                hit = _numbering_overlap(p, t)
                if hit is not None and (best is None or len(hit[0]) > len(best[1][0])):
                    best = (t, hit)
            if best is not None:
                t, (kp, kt) = best
                used_t.add(id(t))
                pr, tr = _restrict(p, kp), _restrict(t, kt)
                groups.setdefault(pr["seq"], ([], []))
                groups[pr["seq"]][0].append(pr), groups[pr["seq"]][1].append(tr)
        groups.pop(seq, None)
    anchors = [(a[0], b[0]) for a, b in groups.values() if a and b]
    if not anchors:
        return []
    # global frame from the first matched pair, then greedy assignment inside each entity
    p0, ok_p = _trace(pred, anchors[0][0])
    t0, ok_t = _trace(true, anchors[0][1])
    both = ok_p & ok_t
    rot, trans = metrics.kabsch(p0[both], t0[both]) if both.sum() >= 3 else (np.eye(3), np.zeros(3))
    for ps, ts in groups.values():
        free = list(ts)
        for p in ps:
            if not free:
                break
            pp, okp = _trace(pred, p)
            pp = pp @ rot.T + trans
            cost = []
            for t in free:
                tq, okt = _trace(true, t)
                m = okp & okt
                cost.append(np.sqrt(((pp[m] - tq[m]) ** 2).sum(-1).mean()) if m.any() else np.inf)
            pairs.append((p, free.pop(int(np.argmin(cost)))))
    return pairs


def matched_atoms(pred, true, pairs):
    """Matched coordinates over all chain pairs: ``(pred xyz, true xyz, chain pair index, residue index, is trace atom)``."""
    px, tx = pred.coords(), true.coords()
    P, T, chain_of, res_of, trace = [], [], [], [], []
    rid = 0
    for k, (p, t) in enumerate(pairs):
        want = b"CA" if p["mol"] == const.MOL_PROTEIN else b"C1'"
        for rp, rt in zip(p["res"], t["res"]):
            ap = pred.atoms[int(rp["atom_idx"]) : int(rp["atom_idx"]) + int(rp["atom_num"])]
            at = true.atoms[int(rt["atom_idx"]) : int(rt["atom_idx"]) + int(rt["atom_num"])]
            where = {a["name"]: j for j, a in enumerate(ap) if a["is_present"]}
            for j, a in enumerate(at):
                i = where.get(a["name"])
                if a["is_present"] and i is not None:
                    P.append(px[int(rp["atom_idx"]) + i]), T.append(tx[int(rt["atom_idx"]) + j])
                    chain_of.append(k), res_of.append(rid)
                    trace.append(a["name"] == want or p["mol"] == const.MOL_NONPOLYMER)
            rid += 1
    return np.array(P).reshape(-1, 3), np.array(T).reshape(-1, 3), np.array(chain_of), np.array(res_of), np.array(trace, bool)


def compare_files(pred_path: str, true_path: str, use_assembly: bool = False) -> dict:
    pred, _ = parse_mmcif(pred_path, use_assembly=False)
    true, _ = parse_mmcif(true_path, use_assembly=use_assembly)
    pairs = match_chains(pred, true)
    if not pairs:
        return {"matched_chains": 0}
    P, T, chain_of, res_of, trace = matched_atoms(pred, true, pairs)
    out = {"matched_chains": len(pairs), "matched_atoms": int(len(P)), "lddt": metrics.lddt(P, T, residue_of=res_of),
           "rmsd_all_atom": metrics.rmsd(P, T)}  # fmt: skip
    if trace.sum() >= 4:
        out["tm_score"] = metrics.tm_score(P[trace], T[trace])
        out["gdt_ts"] = metrics.gdt_ts(P[trace], T[trace])
        out["rmsd_trace"] = metrics.rmsd(P[trace], T[trace])
    # secondary structure from the C-alpha traces of the matched protein chains (residues in chain order)
    from .secondary_structure import ss_agreement

    per_chain, weights = [], []
    for k, (p, _) in enumerate(pairs):
        pick = trace & (chain_of == k)
        if p["mol"] == const.MOL_PROTEIN and int(pick.sum()) >= 8:
            per_chain.append(ss_agreement(P[pick], T[pick]))
            weights.append(int(pick.sum()))
    if per_chain:
        w = np.asarray(weights, float)

        def pooled(key):
            vals = np.asarray([c[key] for c in per_chain], float)
            ok = np.isfinite(vals)
            return float((vals[ok] * w[ok]).sum() / w[ok].sum()) if ok.any() else float("nan")

        out.update(ss_q3=pooled("q3"), ss_f1_helix=pooled("f1_helix"), ss_f1_strand=pooled("f1_strand"))
        rec = [x for c in per_chain for x in c["helix_recovery"]]
        out["helix_recovery"] = float(np.mean(rec)) if rec else float("nan")
    best = None
    for a, b in itertools.combinations(range(len(pairs)), 2):
        ra, rb = chain_of == a, chain_of == b
        if ra.sum() < rb.sum():
            ra, rb = rb, ra  # the larger chain is the receptor
        d = metrics.dockq(P[ra], P[rb], T[ra], T[rb], trace[ra], trace[rb])
        if d["fnat"] > 0 or np.isfinite(d["irmsd"]):
            out.setdefault("interfaces", {})[f"{a}-{b}"] = d
            best = d["dockq"] if best is None else max(best, d["dockq"])
    if out.get("interfaces"):
        out["dockq_mean"] = float(np.mean([d["dockq"] for d in out["interfaces"].values()]))
    return out
