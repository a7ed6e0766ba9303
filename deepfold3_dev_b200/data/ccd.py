"""Chemical component dictionary access without external toolkits (reference: data/ccd.py:40-841, which uses gemmi and
RDKit for ``components.cif`` access, conformer generation, leaving atoms and automorphisms).

``components.cif`` is itself a CIF file: every ``data_<CODE>`` block lists the atoms of one component
(``_chem_comp_atom``: names, elements, formal charges, leaving-atom flags, ideal and model coordinates) and its bonds
(``_chem_comp_bond``). The reference conformer of a component is its ideal coordinate set, falling back to the model
coordinates when the ideal ones are missing - the same fallback order AF3 uses when conformer generation fails.
Hydrogens are dropped. Blocks are located by a streaming scan, so asking for a few codes does not parse the 400 MB file.

Not covered here: generating conformers from SMILES and graph automorphisms of ligands (both need a cheminformatics
toolkit); symmetric atom swaps of standard residues are tabulated in ``data/symmetry.py``.
"""

from __future__ import annotations

import gzip
import json
from dataclasses import dataclass, field

import numpy as np

from . import ref_conformers
from .parse.cif import MISSING, parse_cif
from .parse.mmcif import ATOMIC_NUMBER

_ORDER = {"SING": 1, "DOUB": 2, "TRIP": 3, "AROM": 4}


@dataclass
class Component:
    code: str
    name: str
    atoms: list[str]
    elements: list[int]
    charges: list[int]
    coords: np.ndarray  # [n, 3] ideal (or model) coordinates
    leaving: list[bool]
    bonds: list[tuple[int, int, int]] = field(default_factory=list)  # (atom index, atom index, order; 4 = aromatic)

    def to_table_entry(self) -> dict:
        return {"atoms": self.atoms, "elements": self.elements, "charges": self.charges, "coords": self.coords.round(3).tolist(),
                "leaving": self.leaving, "bonds": [list(b) for b in self.bonds]}  # fmt: skip


def _open(path: str):
    return gzip.open(path, "rt", encoding="utf-8", errors="replace") if str(path).endswith(".gz") else open(path, encoding="utf-8", errors="replace")


def iter_blocks(path: str, codes: set[str] | None = None):
    """Yield ``(code, block text)`` for every (requested) ``data_`` block, reading the file line by line."""
    want = {c.upper() for c in codes} if codes is not None else None
    code, buf, left = None, [], None if want is None else len(want)
    with _open(path) as f:
        for line in f:
            if line.startswith("data_"):
                if code is not None and buf:
                    yield code, "".join(buf)
                    if left is not None:
                        left -= 1
                        if left == 0:
                            return
                code = line[5:].strip().upper()
                buf = [line] if (want is None or code in want) else []
                if not buf:
                    code = None
            elif code is not None:
                buf.append(line)
    if code is not None and buf:
        yield code, "".join(buf)


def _floats(cols: dict, keys: tuple[str, str, str], n: int) -> np.ndarray | None:
    if not all(k in cols for k in keys):
        return None
    out = np.zeros((n, 3), dtype=np.float32)
    for j, k in enumerate(keys):
        for i, v in enumerate(cols[k]):
            if v in MISSING:
                return None
            out[i, j] = float(v)
    return out


def parse_component(text: str, keep_hydrogens: bool = False) -> Component | None:
    block = parse_cif(text)[0]
    a = block.table("chem_comp_atom")
    if not a or "atom_id" not in a:
        return None
    n = len(a["atom_id"])
    xyz = _floats(a, ("pdbx_model_Cartn_x_ideal", "pdbx_model_Cartn_y_ideal", "pdbx_model_Cartn_z_ideal"), n)
    if xyz is None:
        xyz = _floats(a, ("model_Cartn_x", "model_Cartn_y", "model_Cartn_z"), n)
    symbols = a.get("type_symbol", ["C"] * n)
    keep = [i for i in range(n) if keep_hydrogens or symbols[i].upper() not in ("H", "D")]
    index = {a["atom_id"][i].strip('"'): k for k, i in enumerate(keep)}
    charges = a.get("charge", ["0"] * n)
    leaving = a.get("pdbx_leaving_atom_flag", ["N"] * n)
    b = block.table("chem_comp_bond")
    bonds = []
    for x, y, o in zip(b.get("atom_id_1", []), b.get("atom_id_2", []), b.get("value_order", [])):
        i, j = index.get(x.strip('"')), index.get(y.strip('"'))
        if i is not None and j is not None:
            bonds.append((i, j, _ORDER.get(o.upper()[:4], 1)))
    elements = [min(ATOMIC_NUMBER.get(symbols[i].upper(), 6), 127) for i in keep]
    if xyz is None:
        # neither ideal nor model coordinates (a few hundred dictionary entries): embed the heavy-atom graph from its
        # bond list, as the reference does from the entry's SMILES descriptor with a toolkit (data/ccd.py:267-362)
        from .smiles import embed_3d

        aromatic_flag = a.get("pdbx_aromatic_flag", ["N"] * n)
        heavy = embed_3d(elements, bonds, [aromatic_flag[i] == "Y" for i in keep], seed=sum(map(ord, block.name)) % 9973)
        xyz = np.zeros((n, 3), dtype=np.float32)
        xyz[keep] = heavy
    return Component(
        code=block.name.upper(), name=block.value("chem_comp", "name") or "",
        atoms=[a["atom_id"][i].strip('"') for i in keep],
        elements=elements,
        charges=[int(float(charges[i])) if charges[i] not in MISSING else 0 for i in keep],
        coords=xyz[keep], leaving=[leaving[i] == "Y" for i in keep], bonds=bonds,
    )  # fmt: skip


def load_components(path: str, codes: set[str] | None = None) -> dict[str, Component]:
    out = {}
    for code, text in iter_blocks(path, codes):
        comp = parse_component(text)
        if comp is not None and comp.atoms:
            out[code] = comp
    return out


def register(components: dict[str, Component]) -> int:
    """Make the components available to the tokenizers (reference conformers by code)."""
    for code, c in components.items():
        ref_conformers._TABLE[code] = c.to_table_entry()
    return len(components)


def load_ccd(path: str, codes: set[str] | None = None) -> int:
    """``--ccd`` entry point: a JSON conformer table, or ``components.cif[.gz]`` (optionally only some codes)."""
    if str(path).endswith(".json"):
        return ref_conformers.load_table(path)
    return register(load_components(path, codes))


def export_table(path: str, out_json: str, codes: set[str] | None = None) -> int:
    comps = load_components(path, codes)
    with open(out_json, "w") as f:
        json.dump({k: v.to_table_entry() for k, v in comps.items()}, f)
    return len(comps)


def atom_name_sets(components: dict[str, Component]) -> dict[str, set[str]]:
    """Allowed atom names per component (the preparation step drops atoms a component does not define)."""
    return {k: set(v.atoms) for k, v in components.items()}


def leaving_atom_sets(components: dict[str, Component]) -> dict[str, set[str]]:
    return {k: {a for a, flag in zip(v.atoms, v.leaving) if flag} for k, v in components.items()}
