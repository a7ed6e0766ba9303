"""Cluster ids for the manifest's chains.

Reference: data/prepare/clustering.py:21-120 takes protein clusters from wwPDB's ``clusters-by-entity-40.txt`` (one
cluster per line, ``PDB_CHAIN`` members) and keys everything else by sequence hash. Both are here. When no cluster file
is given, proteins are clustered in-process by a greedy k-mer pass (longest first, a chain joins the first
representative with which it shares at least ``identity`` of its 3-mers), which is what an offline box can do without
an external clustering binary; short peptides (< 10 residues), nucleic acids and ligands keep exact-sequence /
component-code keys as AF3 2.5.3 prescribes.
"""

from __future__ import annotations

import hashlib

from .. import const
from ..types import Record


def load_pdb_clusters(path: str) -> dict[str, int]:
    """``clusters-by-entity-40.txt`` -> ``{"1abc_a": cluster index}`` (keys lower-cased)."""
    out: dict[str, int] = {}
    with open(path) as f:
        for k, line in enumerate(f):
            for member in line.split():
                out[member.lower()] = k
    return out


def cluster_key(pdb_id: str, chain_name: str) -> str:
    return f"{pdb_id}_{chain_name}".lower()


def hash_cluster(text: str) -> str:
    return hashlib.sha256(text.encode()).hexdigest()[:16]


def _kmers(seq: str, k: int = 3) -> set[str]:
    return {seq[i : i + k] for i in range(max(len(seq) - k + 1, 1))}


def greedy_kmer_clusters(seqs: dict[str, str], identity: float = 0.4, k: int = 3) -> dict[str, str]:
    """``{key: sequence}`` -> ``{key: representative key}``; deterministic (length, then key order)."""
    order = sorted(seqs, key=lambda key: (-len(seqs[key]), key))
    reps: list[tuple[str, set[str]]] = []
    index: dict[str, list[int]] = {}
    out: dict[str, str] = {}
    for key in order:
        mine = _kmers(seqs[key], k)
        votes: dict[int, int] = {}
        for km in mine:
            for r in index.get(km, ()):
                votes[r] = votes.get(r, 0) + 1
        hit = next((r for r, n in sorted(votes.items()) if n >= identity * len(mine)), None)
        if hit is not None:
            out[key] = reps[hit][0]
            continue
        reps.append((key, mine))
        for km in mine:
            index.setdefault(km, []).append(len(reps) - 1)
        out[key] = key
    return out


def cluster_records(records: list[Record], sequences: dict[str, str] | None = None, pdb_clusters: dict[str, int] | None = None,
                    identity: float = 0.4) -> list[Record]:  # fmt: skip
    """Fill ``cluster_id`` of every chain in place.

    ``sequences`` maps ``msa_id`` -> one-letter sequence for polymer chains (as written by the preparation step).
    """
    sequences = sequences or {}
    prot = {}
    for rec in records:
        for ci in rec.chains:
            seq = sequences.get(str(ci.msa_id))
            if ci.mol_type == const.MOL_PROTEIN and seq and len(seq) >= 10:
                prot[str(ci.msa_id)] = seq
    rep_of = greedy_kmer_clusters(prot, identity) if (prot and pdb_clusters is None) else {}
    for rec in records:
        for ci in rec.chains:
            if ci.mol_type == const.MOL_NONPOLYMER:
                ci.cluster_id = f"lig:{ci.res_name or ci.msa_id}"
                continue
            if pdb_clusters is not None and ci.mol_type == const.MOL_PROTEIN:
                hit = pdb_clusters.get(cluster_key(rec.id, ci.auth_chain_name or ci.chain_name))
                if hit is not None:
                    ci.cluster_id = hit
                    continue
            ci.cluster_id = rep_of.get(str(ci.msa_id), hash_cluster(sequences.get(str(ci.msa_id), str(ci.msa_id))))
    return records
