"""A3M alignment parser (reference: data/parse/a3m.py).

Lower-case letters are insertions relative to the query: they are removed from the aligned row and
counted into the deletion value of the next aligned column. ``-`` is a gap, ``.`` is ignored.
"""

from __future__ import annotations

import dataclasses

import numpy as np

from .. import const


@dataclasses.dataclass
class MSA:
    sequences: list[str]  # aligned rows, all of the query's length (row 0 = query)
    deletions: np.ndarray  # [S, N] int32
    descriptions: list[str]

    def __len__(self):
        return len(self.sequences)


def read_fasta_like(text: str) -> tuple[list[str], list[str]]:
    names, seqs, cur = [], [], []
    for line in text.splitlines():
        line = line.strip()
        if not line or line.startswith("#"):
            continue
        if line.startswith(">"):
            if cur or names:
                seqs.append("".join(cur))
            names.append(line[1:])
            cur = []
        else:
            cur.append(line.replace("\x00", ""))
    if names:
        seqs.append("".join(cur))
    return names, seqs


def parse_a3m(text: str, max_rows: int | None = None, dedup: bool = True) -> MSA:
    names, raw = read_fasta_like(text)
    if not raw:
        raise ValueError("empty A3M")
    n = sum(1 for c in raw[0] if not c.islower() and c != ".")
    rows, dels, descs, seen = [], [], [], set()
    for name, seq in zip(names, raw):
        aligned, row_del, pending = [], [], 0
        for c in seq:
            if c == ".":
                continue
            if c.islower():
                pending += 1
            else:
                aligned.append(c)
                row_del.append(pending)
                pending = 0
        if len(aligned) != n:
            # concatenated search results can leave a row with a second block glued on (a lost header) or cut short:
            # keep the first n columns, fill a short row with gaps (same outcome as the reference's fixed-width fill)
            aligned, row_del = aligned[:n], row_del[:n]
            row_del += [0] * (n - len(aligned))
            aligned += ["-"] * (n - len(aligned))
        s = "".join(aligned)
        if dedup and s in seen:
            continue
        seen.add(s)
        rows.append(s)
        dels.append(row_del)
        descs.append(name)
        if max_rows is not None and len(rows) >= max_rows:
            break
    return MSA(rows, np.asarray(dels, dtype=np.int32).reshape(len(rows), n), descs)


_PROT = {c: const.RES_TYPE_ORDER[n3] for c, n3 in const.PROTEIN_1TO3.items()}
_RNA = {c: const.RES_TYPE_ORDER[n] for c, n in const.RNA_1TO3.items()}
_DNA = {c: const.RES_TYPE_ORDER[n] for c, n in const.DNA_1TO3.items()}


def encode_sequence(seq: str, mol_type: int) -> np.ndarray:
    """Residue-type ids of an aligned row; gaps map to ``MSA_GAP``, unknown letters to the type's unknown id."""
    table = {const.MOL_PROTEIN: _PROT, const.MOL_RNA: _RNA, const.MOL_DNA: _DNA}[mol_type]
    unk = const.RES_TYPE_ORDER["UNK"] if mol_type == const.MOL_PROTEIN else const.RES_TYPE_ORDER["N"]
    return np.asarray([const.MSA_GAP if c == "-" else table.get(c.upper(), unk) for c in seq], dtype=np.int64)


def msa_from_a3m_file(path: str, mol_type: int, max_rows: int | None = None):
    """A3M file -> the array form stored next to prepared structures (``data.types.MSA``: int8 rows, mask, deletions)."""
    from ..types import MSA as ArrayMSA

    from ..io_cache import read_text

    m = parse_a3m(read_text(path), max_rows=max_rows)
    rows = np.stack([encode_sequence(s, mol_type) for s in m.sequences]).astype(np.int8)
    return ArrayMSA(rows, rows != const.MSA_GAP, np.clip(m.deletions, 0, 127).astype(np.int8))
