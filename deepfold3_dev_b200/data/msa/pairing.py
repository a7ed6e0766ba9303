"""Species pairing of per-chain alignments (reference: data/msa/pairing.py:55-270).

Rows of different chains are joined into one complex row when they come from the same species. The species of a
row is read from its A3M header: UniProt style ``OX=<taxid>`` / ``TaxID=<taxid>`` tags, or the mnemonic after the
underscore of ``tr|ACC|NAME_SPECIES``. Within a species the k-th best hits of every chain are paired (hits keep
their search order), and species are ordered by how many chains they cover, then by rank.
"""

from __future__ import annotations

import dataclasses
import re
from collections.abc import Sequence

import numpy as np

from ..parse.a3m import MSA

_OX = re.compile(r"(?:OX|TaxID)=(\d+)")
_MNEMONIC = re.compile(r"^(?:sp|tr)\|[^|]*\|\w+_(\w+)")


def species_id(header: str) -> str:
    m = _OX.search(header)
    if m:
        return m.group(1)
    m = _MNEMONIC.match(header.strip())
    return m.group(1) if m else ""


def species_ids(headers: Sequence[str]) -> np.ndarray:
    return np.asarray([species_id(h) for h in headers], dtype=object)


def species_fraction(species: np.ndarray | None) -> float:
    if species is None or len(species) == 0:
        return 0.0
    return float(np.mean([bool(s) for s in species]))


@dataclasses.dataclass
class PairingResult:
    rows: np.ndarray  # [P, chains] row index into each chain's alignment, -1 where the chain has no partner
    species: list


def find_pairing_indices(per_chain_species: list[np.ndarray], max_rows: int = 8191, min_chains: int = 2) -> PairingResult:
    """Row indices that pair up; row 0 of every chain (the query) is always the first paired row."""
    n = len(per_chain_species)
    by_species: dict[str, list[list[int]]] = {}
    for c, sp in enumerate(per_chain_species):
        for i, s in enumerate(sp):
            if i == 0 or not s:
                continue
            by_species.setdefault(s, [[] for _ in range(n)])[c].append(i)
    rows, names = [[0] * n], ["query"]
    ranked = sorted(by_species.items(), key=lambda kv: (-sum(bool(x) for x in kv[1]), min(x[0] for x in kv[1] if x)))
    for name, hits in ranked:
        covered = sum(bool(x) for x in hits)
        if covered < min_chains:
            continue
        depth = max(len(x) for x in hits)
        for k in range(depth):
            row = [hits[c][k] if k < len(hits[c]) else -1 for c in range(n)]
            if sum(r >= 0 for r in row) >= min_chains:
                rows.append(row)
                names.append(name)
            if len(rows) >= max_rows:
                break
        if len(rows) >= max_rows:
            break
    return PairingResult(np.asarray(rows, dtype=np.int64), names)


def pair_by_species(msas: list[MSA], max_rows: int = 8191) -> tuple[list[MSA], PairingResult]:
    """Paired alignments (one per chain, equal depth, gaps where a chain has no partner) and the pairing itself."""
    res = find_pairing_indices([species_ids(m.descriptions) for m in msas], max_rows)
    out = []
    for c, m in enumerate(msas):
        width = len(m.sequences[0])
        seqs, dels, descs = [], [], []
        for r in res.rows[:, c]:
            if r >= 0:
                seqs.append(m.sequences[r])
                dels.append(m.deletions[r])
                descs.append(m.descriptions[r])
            else:
                seqs.append("-" * width)
                dels.append(np.zeros(width, dtype=np.int32))
                descs.append("")
        out.append(MSA(seqs, np.stack(dels), descs))
    return out, res


def unpaired_rows_not_in_paired(unpaired: MSA, paired: MSA) -> np.ndarray:
    """Indices of the unpaired alignment whose sequence does not already occur among the paired rows."""
    seen = set(paired.sequences)
    return np.asarray([i for i, s in enumerate(unpaired.sequences) if i == 0 or s not in seen], dtype=np.int64)
