"""``Structure`` record arrays <-> mmCIF text, and predicted coordinates -> ``Structure``.

Reference: io/structure_mmcif.py (a parsed structure written back as mmCIF) and io/structure_builder.py (model output
placed into a ``Structure``). The text written here carries what the reader in ``data/parse/mmcif.py`` consumes:
``_entity``, ``_entity_poly``, ``_entity_poly_seq``, ``_struct_asym``, ``_atom_site`` (resolved atoms only, B-factor
column kept) and ``_struct_conn`` for bonds between residues, so a structure survives a write / read cycle.
"""

from __future__ import annotations

import numpy as np

from ..data import const
from ..data.parse.mmcif import _PERIODIC
from ..data.types import Structure

_POLY_TYPE = {const.MOL_PROTEIN: "polypeptide(L)", const.MOL_DNA: "polydeoxyribonucleotide", const.MOL_RNA: "polyribonucleotide"}


def _q(v: str) -> str:
    v = str(v)
    if not v:
        return "?"
    return f'"{v}"' if any(c in v for c in " '#") or v[0] in "_;$[]" else v


def structure_to_mmcif(st: Structure, entry_id: str | None = None) -> str:
    name = entry_id or st.name or "structure"
    out = [f"data_{name}", f"_entry.id {name}", "#"]
    entities: dict[int, int] = {}
    for c in st.chains:
        entities.setdefault(int(c["entity_id"]), int(c["asym_id"]))
    out += ["loop_", "_entity.id", "_entity.type"]
    for e, a in entities.items():
        out.append(f"{e + 1} {'polymer' if int(st.chains[a]['mol_type']) != const.MOL_NONPOLYMER else 'non-polymer'}")
    poly = {e: a for e, a in entities.items() if int(st.chains[a]["mol_type"]) != const.MOL_NONPOLYMER}
    if poly:
        out += ["#", "loop_", "_entity_poly.entity_id", "_entity_poly.type", "_entity_poly.pdbx_seq_one_letter_code_can"]
        for e, a in poly.items():
            seq = (st.chain_canonical_seqs or {}).get(a, "?")
            out.append(f"{e + 1} {_q(_POLY_TYPE[int(st.chains[a]['mol_type'])])} {seq}")
        out += ["#", "loop_", "_entity_poly_seq.entity_id", "_entity_poly_seq.num", "_entity_poly_seq.mon_id"]
        for e, a in poly.items():
            c = st.chains[a]
            for k, r in enumerate(st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]):
                out.append(f"{e + 1} {k + 1} {r['name'].decode().strip()}")
    out += ["#", "loop_", "_struct_asym.id", "_struct_asym.entity_id"]
    labels = {}
    for c in st.chains:
        labels[int(c["asym_id"])] = c["name"].decode().strip() or f"C{int(c['asym_id'])}"
    if len(set(labels.values())) < len(labels):  # chain names must be unique as label ids
        labels = {a: f"{n}{a}" for a, n in labels.items()}
    for c in st.chains:
        out.append(f"{labels[int(c['asym_id'])]} {int(c['entity_id']) + 1}")
    cols = ("group_PDB id type_symbol label_atom_id label_alt_id label_comp_id label_asym_id label_entity_id label_seq_id "
            "Cartn_x Cartn_y Cartn_z occupancy B_iso_or_equiv pdbx_formal_charge auth_seq_id auth_asym_id pdbx_PDB_model_num").split()  # fmt: skip
    out += ["#", "loop_"] + [f"_atom_site.{c}" for c in cols]
    serial = 0
    where: dict[int, tuple[str, str, str, str]] = {}
    for c in st.chains:
        lab, ent, mt = labels[int(c["asym_id"])], int(c["entity_id"]) + 1, int(c["mol_type"])
        for k, r in enumerate(st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]):
            comp = r["name"].decode().strip()
            seq = str(k + 1) if mt != const.MOL_NONPOLYMER else "."
            for i in range(int(r["atom_idx"]), int(r["atom_idx"]) + int(r["atom_num"])):
                a = st.atoms[i]
                if not a["is_present"]:
                    continue
                serial += 1
                z = int(a["element"])
                sym = _PERIODIC[z - 1].upper() if 1 <= z <= len(_PERIODIC) else "X"
                an = a["name"].decode().strip()
                where[i] = (lab, comp, seq if seq != "." else str(int(r["res_id"])), an)
                out.append(f"{'ATOM' if mt != const.MOL_NONPOLYMER else 'HETATM'} {serial} {sym} {_q(an)} . {comp} {lab} {ent} {seq} "
                           f"{a['x']:.3f} {a['y']:.3f} {a['z']:.3f} 1.00 {a['b_factor']:.2f} {int(a['charge'])} {int(r['res_id'])} {lab} 1")  # fmt: skip
    res_of = np.repeat(np.arange(len(st.residues)), st.residues["atom_num"]) if len(st.residues) else np.zeros(0, int)
    links = [(int(b["atom_1"]), int(b["atom_2"])) for b in st.bonds
             if int(b["atom_1"]) in where and int(b["atom_2"]) in where and res_of[int(b["atom_1"])] != res_of[int(b["atom_2"])]]  # fmt: skip
    if links:
        out += ["#", "loop_"] + [f"_struct_conn.{c}" for c in (
            "id conn_type_id ptnr1_label_asym_id ptnr1_label_comp_id ptnr1_label_seq_id ptnr1_auth_seq_id ptnr1_label_atom_id "
            "ptnr2_label_asym_id ptnr2_label_comp_id ptnr2_label_seq_id ptnr2_auth_seq_id ptnr2_label_atom_id").split()]  # fmt: skip
        for n, (i, j) in enumerate(links):
            (l1, c1, s1, a1), (l2, c2, s2, a2) = where[i], where[j]
            out.append(f"covale{n + 1} covale {l1} {c1} {s1} {s1} {_q(a1)} {l2} {c2} {s2} {s2} {_q(a2)}")
    return "\n".join(out) + "\n#\n"


def write_structure(st: Structure, path: str) -> None:
    with open(path, "w") as f:
        f.write(structure_to_mmcif(st))


def with_coordinates(st: Structure, token_atom_positions, atom_rows, b_factors=None) -> Structure:
    """Copy of ``st`` whose atoms take model output: ``token_atom_positions`` [N, 24, 3] indexed through ``atom_rows``
    (per token, the rows of ``st.atoms`` it covers, as returned by ``featurize.tokenize_structure``)."""
    atoms = st.atoms.copy()
    pos = np.asarray(token_atom_positions, dtype=np.float32)
    for t, rows in enumerate(atom_rows):
        k = len(rows)
        atoms["x"][rows], atoms["y"][rows], atoms["z"][rows] = pos[t, :k, 0], pos[t, :k, 1], pos[t, :k, 2]
        atoms["is_present"][rows] = True
        if b_factors is not None:
            atoms["b_factor"][rows] = np.asarray(b_factors, dtype=np.float32)[t, :k]
    return Structure(atoms, st.bonds, st.residues, st.chains, st.name, st.chain_canonical_seqs)
