"""Reference conformers of residues and ligands (the ``ref_pos`` / ``ref_element`` / ``ref_charge`` features).

The reference builds them from the wwPDB chemical component dictionary with gemmi / RDKit
(data/feature/ref_atoms.py:138-250, data/ccd.py). Neither is available offline, so conformers come from

1. a user table (``load_table``: JSON ``{name: {"atoms": [...], "elements": [...], "charges": [...],
   "coords": [[x, y, z], ...]}}``, e.g. exported once from the CCD), else
2. a built-in generator for the standard residues: backbone atoms at the standard peptide geometry,
   side-chain and nucleotide atoms laid out along the bonded chain in ``const.RESIDUE_ATOMS`` order at
   1.5 Angstrom spacing with a fixed zig-zag. The atom set, names, elements and ordering are exact; the
   side-chain geometry is schematic. Single ions are one atom at the origin.
"""

from __future__ import annotations

import json
import math

import numpy as np

from . import const

_TABLE: dict[str, dict] = {}
_BACKBONE = {"N": (-0.525, 1.363, 0.0), "CA": (0.0, 0.0, 0.0), "C": (1.526, 0.0, 0.0), "O": (2.153, -1.062, 0.0),
             "CB": (-0.529, -0.774, -1.205)}  # fmt: skip
IONS = {"MG", "ZN", "FE", "CA", "NA", "K", "MN", "CU", "CO", "NI", "CL", "BR", "I", "F"}


def load_table(path: str) -> int:
    with open(path) as f:
        data = json.load(f)
    for name, rec in data.items():
        _TABLE[name.upper()] = rec
    return len(data)


CCD_PATH: str | None = None  # components.cif[.gz]; looked up lazily, one streaming pass per batch of missing codes


def set_ccd_source(path: str | None) -> None:
    """A ``.json`` conformer table is loaded at once; ``components.cif[.gz]`` is remembered and read on demand."""
    global CCD_PATH
    if path and str(path).endswith(".json"):
        load_table(path)
    else:
        CCD_PATH = path


def ensure_components(codes) -> None:
    """Load the listed component codes from the dictionary file if they are not known yet."""
    missing = {c.upper() for c in codes if c and c.upper() not in _TABLE and c.upper() not in const.RESIDUE_ATOMS}
    if missing and CCD_PATH:
        from . import ccd

        ccd.register(ccd.load_components(CCD_PATH, missing))


def load_component_text(text: str) -> int:
    """Custom components given inline as CIF text (the ``userCCD`` field of a prediction job)."""
    from . import ccd

    found = {}
    for block in text.split("\ndata_"):
        block = block if block.startswith("data_") else "data_" + block
        comp = ccd.parse_component(block)
        if comp is not None and comp.atoms:
            found[comp.code] = comp
    return ccd.register(found)


def _zigzag(start, n: int, step: float = 1.5):
    """``n`` points leaving ``start`` along -z with alternating lateral offsets (a schematic carbon chain)."""
    pts, p = [], np.asarray(start, dtype=np.float64)
    for i in range(n):
        p = p + np.asarray([0.6 * step * (1 if i % 2 else -1), 0.35 * step * math.cos(i), -0.75 * step])
        pts.append(p.copy())
    return pts


def get_ref_atoms(res_name: str):
    """``(atom_names, elements, charges, coords[n, 3])`` of a component, or ``None`` if it is unknown."""
    name = res_name.upper()
    rec = _TABLE.get(name)
    if rec is not None:
        atoms = list(rec["atoms"])
        elements = [const.ELEMENT_NUMBER.get(str(e).upper(), 6) if not isinstance(e, int) else e for e in rec["elements"]]
        charges = list(rec.get("charges", [0] * len(atoms)))
        return atoms, elements, charges, np.asarray(rec["coords"], dtype=np.float32).reshape(len(atoms), 3)
    if name in const.RESIDUE_ATOMS:
        atoms = list(const.RESIDUE_ATOMS[name])
        coords = []
        if atoms[0] == "N":  # amino acid
            side = [a for a in atoms if a not in _BACKBONE]
            chain = _zigzag(_BACKBONE["CB"], len(side))
            it = iter(chain)
            coords = [_BACKBONE[a] if a in _BACKBONE else tuple(next(it)) for a in atoms]
        else:  # nucleotide: one chain from the phosphate
            coords = [(0.0, 0.0, 0.0)] + [tuple(p) for p in _zigzag((0.0, 0.0, 0.0), len(atoms) - 1)]
        elements = [const.atom_element(a) for a in atoms]
        return atoms, elements, [0] * len(atoms), np.asarray(coords, dtype=np.float32)
    if name in IONS:
        return [name], [const.ELEMENT_NUMBER[name]], [0], np.zeros((1, 3), dtype=np.float32)
    return None
