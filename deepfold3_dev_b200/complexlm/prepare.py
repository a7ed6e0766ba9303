"""Store builders of the complex language model (reference: complexlm/prepare.py, cluster.py; ``plm-prepare`` command).

``structure``: a directory of prepared structures (``structures/*.npz`` + ``manifest.json``) -> store with per-residue
interface flags (any heavy atom within 5 A of another chain). ``pairs``: FASTA + a list of id pairs -> two-chain
complexes without interface labels. ``cluster``: complex-level cluster ids over several stores at once from chain
clusters (a complex's key is the sorted set of its chains' cluster ids); chain clusters use the in-process k-mer
clustering of the preparation package. ``stats``: size summary.
"""

from __future__ import annotations

import hashlib
import json
import os

import numpy as np

from ..data import const
from .data import ComplexStore, ComplexStoreWriter
from .model import decode


def _one_letter(st, chain_row) -> str:
    letters = {v: k for k, v in const.PROTEIN_1TO3.items()}
    res = st.residues[int(chain_row["res_idx"]) : int(chain_row["res_idx"]) + int(chain_row["res_num"])]
    return "".join(letters.get(const.RES_TYPE_INDEX_TO_NAME.get(int(t), "UNK"), "X") for t in res["res_type"])


def interface_flags(st, protein_chains: list[int], cutoff: float = 5.0) -> list[np.ndarray]:
    """Per protein chain, per residue: does any resolved atom lie within ``cutoff`` of another chain's atom."""
    from scipy.spatial import cKDTree

    xyz = st.coords().astype(np.float64)
    present = st.atoms["is_present"]
    chain_pts = {}
    for c in st.chains:
        sl = st.chain_atoms(c)
        chain_pts[int(c["asym_id"])] = xyz[sl][present[sl]]
    trees = {a: cKDTree(p) for a, p in chain_pts.items() if len(p)}
    out = []
    for a in protein_chains:
        c = st.chains[a]
        res = st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]
        flags = np.zeros(len(res), np.uint8)
        for k, r in enumerate(res):
            rows = np.arange(int(r["atom_idx"]), int(r["atom_idx"]) + int(r["atom_num"]))
            pts = xyz[rows][present[rows]]
            if not len(pts):
                continue
            for b, tree in trees.items():
                if b != a and np.isfinite(tree.query(pts, distance_upper_bound=cutoff)[0]).any():
                    flags[k] = 1
                    break
        out.append(flags)
    return out


def build_from_structures(data_dir: str, output: str, source: str, min_len: int = 8) -> dict:
    from ..data.types import Structure, load_manifest

    w = ComplexStoreWriter(output, source, with_iface=True)
    for rec in load_manifest(os.path.join(data_dir, "manifest.json")):
        st = Structure.load(os.path.join(data_dir, "structures", f"{rec.id}.npz"))
        prot = [c.chain_id for c in rec.chains if c.valid and c.mol_type == const.MOL_PROTEIN and c.num_residues >= min_len]
        if not prot:
            continue
        released = (rec.structure_info.released if rec.structure_info else None) or ""
        date = int(released.replace("-", "")) if released.replace("-", "").isdigit() else 0
        w.add(rec.id, [_one_letter(st, st.chains[a]) for a in prot], interface_flags(st, prot), date)
    return w.close()


def build_from_pairs(fasta: str, pairs: str, output: str, source: str) -> dict:
    from ..data.prepare.pipeline import load_fasta

    seqs = load_fasta(fasta)
    w = ComplexStoreWriter(output, source, with_iface=False)
    with open(pairs) as f:
        for line in f:
            ids = line.split()
            if len(ids) >= 2 and all(i in seqs for i in ids[:2]):
                w.add("-".join(ids[:2]), [seqs[ids[0]], seqs[ids[1]]])
    return w.close()


def cluster_stores(roots: list[str], identity: float = 0.4) -> dict:
    """Chain clusters across all stores, then complex clusters; ids are written back into each store."""
    from ..data.prepare.clustering import greedy_kmer_clusters

    stores = [ComplexStore(r) for r in roots]
    seqs = {}
    for si, s in enumerate(stores):
        for row in range(len(s.chain_off) - 1):
            seqs[(si, row)] = decode(s.seq[s.chain_off[row] : s.chain_off[row + 1]])
    rep = greedy_kmer_clusters({f"{a}:{b}": v for (a, b), v in seqs.items()}, identity)
    rep_id = {r: i for i, r in enumerate(sorted(set(rep.values())))}
    run = hashlib.sha1(json.dumps(sorted(roots)).encode()).hexdigest()[:12]
    cx_key: dict[tuple, int] = {}
    for si, s in enumerate(stores):
        chain_cluster = np.array([rep_id[rep[f"{si}:{row}"]] for row in range(len(s.chain_off) - 1)], dtype=np.int32)
        cx_cluster = np.zeros(len(s), dtype=np.int32)
        for i in range(len(s)):
            rows = np.asarray(s.slot_chain[s.cx_off[i] : s.cx_off[i + 1]])
            key = tuple(sorted(set(chain_cluster[rows].tolist())))
            cx_cluster[i] = cx_key.setdefault(key, len(cx_key))
        np.save(os.path.join(s.root, "chain_cluster.npy"), chain_cluster)
        np.save(os.path.join(s.root, "cx_cluster.npy"), cx_cluster)
        meta = dict(s.meta, cluster_run=run)
        with open(os.path.join(s.root, "meta.json"), "w") as f:
            json.dump(meta, f, indent=1)
    return {"chain_clusters": len(rep_id), "complex_clusters": len(cx_key), "cluster_run": run}


def store_stats(root: str) -> dict:
    s = ComplexStore(root)
    ent, nch = s.n_entities(), s.n_chains()
    return {"source": s.name, "complexes": len(s), "unique_chains": len(s.chain_off) - 1, "residues": int(len(s.seq)),
            "homomers": int(((ent == 1) & (nch > 1)).sum()), "heteromers": int((ent > 1).sum()), "monomers": int((nch == 1).sum()),
            "dated": int((np.asarray(s.cx_date) > 0).sum()), "has_iface": s.has_iface}  # fmt: skip
