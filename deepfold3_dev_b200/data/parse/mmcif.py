"""mmCIF entry -> ``Structure`` + manifest ``Record``.

Follows what the reference's preparation step produces (data/prepare/structure.py:589-1080, which goes through gemmi):
first model only, hydrogens and waters removed, one alternate location per atom (highest occupancy), polymer chains
laid out on the full ``_entity_poly_seq`` sequence with unresolved residues kept as absent atoms, standard residues
in dense chemical-component atom order, modified residues mapped to their parents for typing, ligands as one chain per
``label_asym_id``, biological assembly 1 expanded from ``_pdbx_struct_assembly_gen`` / ``_pdbx_struct_oper_list``,
entity ids from the canonical sequence, chain-chain interfaces at 5 A, sha256 sequence hashes as MSA / cluster keys.
Bonds: ``_struct_conn`` covalent links, plus intra-residue bonds of non-standard components from ``_chem_comp_bond``
when the file carries it and otherwise from covalent-radius distances.
"""

from __future__ import annotations

import hashlib
import itertools
import os
import re

import numpy as np

from .. import const
from ..types import ATOM_DTYPE, BOND_DTYPE, CHAIN_DTYPE, RESIDUE_DTYPE, ChainInfo, InterfaceInfo, Record, Structure, StructureInfo
from .cif import MISSING, CifBlock, read_cif

INTERFACE_CUTOFF = 5.0
WATER = frozenset({"HOH", "DOD", "WAT", "H2O"})
# modified / alternative names typed as their parent (the hash of a chain uses the parent names too)
PARENT = {"MSE": "MET", "ASX": "ASP", "GLX": "GLU", "SEC": "CYS", "PYL": "LYS", "HSD": "HIS", "HSE": "HIS", "HSP": "HIS",
          "HIE": "HIS", "HID": "HIS", "HIP": "HIS", "CYX": "CYS", "SEP": "SER", "TPO": "THR", "PTR": "TYR", "MLY": "LYS",
          "M3L": "LYS", "HYP": "PRO", "CSO": "CYS", "KCX": "LYS", "5MC": "C", "PSU": "U", "OMG": "G", "OMC": "C",
          "1MA": "A", "2MG": "G", "5MU": "U", "H2U": "U", "7MG": "G", "M2G": "G", "5CM": "DC", "8OG": "DG"}  # fmt: skip
_POLY_KIND = (("polypeptide", const.MOL_PROTEIN), ("polydeoxyribonucleotide/polyribonucleotide", const.MOL_RNA),
              ("polydeoxyribonucleotide", const.MOL_DNA), ("polyribonucleotide", const.MOL_RNA))  # fmt: skip
_PERIODIC = ("H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y "
             "Zr Nb Mo Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re "
             "Os Ir Pt Au Hg Tl Pb Bi Po At Rn").split()  # fmt: skip
ATOMIC_NUMBER = {s.upper(): i + 1 for i, s in enumerate(_PERIODIC)}
_RADIUS = {1: 0.31, 5: 0.84, 6: 0.76, 7: 0.71, 8: 0.66, 9: 0.57, 14: 1.11, 15: 1.07, 16: 1.05, 17: 1.02, 34: 1.20,
           35: 1.20, 53: 1.39}  # fmt: skip
_BOND_ORDER = {"SING": 1, "DOUB": 2, "TRIP": 3, "AROM": 4}


def mol_type_of_polymer(poly_type: str) -> int | None:
    """``_entity_poly.type`` -> molecule class (hybrid DNA/RNA counts as RNA; peptide nucleic acid etc. -> None)."""
    t = poly_type.lower()
    for key, mt in _POLY_KIND:
        if t.startswith(key):
            return mt
    return None


def residue_type(name: str, mol_type: int) -> tuple[int, bool]:
    """(index in the 31-class residue vocabulary, is-standard) for a component name."""
    if name in const.RES_TYPE_ORDER and name not in ("-",):
        return const.RES_TYPE_ORDER[name], name not in ("UNK", "N")
    parent = PARENT.get(name)
    if parent in const.RES_TYPE_ORDER:
        return const.RES_TYPE_ORDER[parent], False
    if mol_type in (const.MOL_DNA, const.MOL_RNA):
        return const.RES_TYPE_ORDER["N"], False
    return const.RES_TYPE_ORDER["UNK"], False


def _element(symbol: str, atom_name: str) -> int:
    s = symbol.upper()
    if s in ATOMIC_NUMBER:
        return min(ATOMIC_NUMBER[s], 127)
    head = re.sub(r"[^A-Za-z]", "", atom_name).upper()
    return min(ATOMIC_NUMBER.get(head[:2], ATOMIC_NUMBER.get(head[:1], 6)), 127)


def sequence_hash(key: str) -> str:
    return hashlib.sha256(key.encode()).hexdigest()


# ---------------------------------------------------------------------------------------------------------------
# metadata
# ---------------------------------------------------------------------------------------------------------------
def structure_info(block: CifBlock) -> StructureInfo:
    res = None
    for cat, item in (("refine", "ls_d_res_high"), ("em_3d_reconstruction", "resolution"), ("reflns", "d_resolution_high")):
        v = block.value(cat, item)
        if v is not None:
            try:
                res = float(v)
                break
            except ValueError:
                pass
    hist = block.table("pdbx_audit_revision_history")
    released = min((d for d in hist.get("revision_date", []) if d not in MISSING), default=None)
    deposited = block.value("pdbx_database_status", "recvd_initial_deposition_date")
    return StructureInfo(resolution=res, method=block.value("exptl", "method"), deposited=deposited,
                         released=released or deposited)  # fmt: skip


def read_structure_info(path: str) -> StructureInfo | None:
    """Metadata only (cheap scan used by ``scan-mmcif``); ``None`` when the file cannot be read."""
    try:
        return structure_info(read_cif(path)[0])
    except Exception:  # noqa: BLE001 - a scan reports unreadable files instead of stopping
        return None


# ---------------------------------------------------------------------------------------------------------------
# assembly operators
# ---------------------------------------------------------------------------------------------------------------
def _expand_ids(expr: str) -> list[str]:
    out: list[str] = []
    for part in expr.split(","):
        part = part.strip()
        m = re.fullmatch(r"(\d+)-(\d+)", part)
        out.extend(str(i) for i in range(int(m.group(1)), int(m.group(2)) + 1)) if m else out.append(part)
    return [p for p in out if p]


def parse_oper_expression(expr: str) -> list[list[str]]:
    """``"(1-3)(4,5)"`` -> ``[[1,4],[1,5],[2,4],...]``: each entry lists the operators applied right to left."""
    groups = re.findall(r"\(([^()]*)\)", expr)
    groups = groups or [expr]
    return [list(combo) for combo in itertools.product(*[_expand_ids(g) for g in groups])]


def assembly_operations(block: CifBlock, assembly_id: str = "1"):
    """``[(asym_id, 4x4 matrix, is_identity)]`` for one assembly; ``None`` when the entry defines none."""
    ops = block.table("pdbx_struct_oper_list")
    gen = block.table("pdbx_struct_assembly_gen")
    if not ops or not gen:
        return None
    mats: dict[str, np.ndarray] = {}
    for r, oid in enumerate(ops["id"]):
        m = np.eye(4)
        try:
            for i in range(3):
                for j in range(3):
                    m[i, j] = float(ops[f"matrix[{i + 1}][{j + 1}]"][r])
                m[i, 3] = float(ops[f"vector[{i + 1}]"][r])
        except (KeyError, ValueError):
            pass
        mats[oid] = m
    out = []
    for r, aid in enumerate(gen["assembly_id"]):
        if aid != assembly_id:
            continue
        for combo in parse_oper_expression(gen["oper_expression"][r]):
            m = np.eye(4)
            for oid in combo:
                m = m @ mats.get(oid, np.eye(4))
            ident = bool(np.allclose(m, np.eye(4), atol=1e-6))
            for asym in gen["asym_id_list"][r].split(","):
                out.append((asym.strip(), m, ident))
    return out or None


# ---------------------------------------------------------------------------------------------------------------
# the builder
# ---------------------------------------------------------------------------------------------------------------
def _atom_rows(block: CifBlock):
    """Per ``label_asym_id``: ordered residue keys and the chosen atom rows (first model, no H, no water, one altloc)."""
    t = block.table("atom_site")
    if not t:
        raise ValueError("no _atom_site category")
    n = len(t["label_asym_id"] if "label_asym_id" in t else t["auth_asym_id"])
    col = lambda k, d=".": t.get(k) or [d] * n  # noqa: E731
    asym, comp, atom = col("label_asym_id"), col("label_comp_id"), col("label_atom_id")
    if "label_asym_id" not in t:
        asym = col("auth_asym_id")
    seq, aseq, ins = col("label_seq_id"), col("auth_seq_id"), col("pdbx_PDB_ins_code")
    sym, alt, occ = col("type_symbol", ""), col("label_alt_id"), col("occupancy", "1.0")
    xs, ys, zs, bf = col("Cartn_x"), col("Cartn_y"), col("Cartn_z"), col("B_iso_or_equiv", "0")
    chg, model, auth = col("pdbx_formal_charge", "0"), col("pdbx_PDB_model_num", "1"), col("auth_asym_id")
    first_model = model[0] if n else "1"
    chains: dict[str, dict] = {}
    for i in range(n):
        if model[i] != first_model:
            break
        if comp[i] in WATER or sym[i].upper() in ("H", "D"):
            continue
        name = atom[i].strip('"')
        if not sym[i] and name[:1] in ("H", "D") and comp[i] in const.RESIDUE_ATOMS:
            continue
        ch = chains.setdefault(asym[i], {"auth": auth[i], "order": [], "res": {}})
        key = (seq[i] if seq[i] not in MISSING else aseq[i], ins[i] if ins[i] not in MISSING else "")
        res = ch["res"].get(key)
        if res is None:
            res = ch["res"][key] = {"comp": comp[i], "auth_seq": aseq[i], "atoms": {}}
            ch["order"].append(key)
        if comp[i] != res["comp"]:  # microheterogeneity: the first listed component wins
            continue
        try:
            o = float(occ[i])
        except ValueError:
            o = 1.0
        old = res["atoms"].get(name)
        if old is not None and (alt[i] in MISSING or o <= old[0]):
            continue
        try:
            q = float(chg[i]) if chg[i] not in MISSING else 0.0
        except ValueError:
            q = 0.0
        res["atoms"][name] = (o, float(xs[i]), float(ys[i]), float(zs[i]), _element(sym[i], name), q,
                              float(bf[i]) if bf[i] not in MISSING else 0.0)  # fmt: skip
    return chains


def _entities(block: CifBlock):
    kind = dict(zip(block.column("entity", "id"), (k.lower() for k in block.column("entity", "type"))))
    asym_entity = dict(zip(block.column("struct_asym", "id"), block.column("struct_asym", "entity_id")))
    poly_type = dict(zip(block.column("entity_poly", "entity_id"), block.column("entity_poly", "type")))
    one_letter = dict(zip(block.column("entity_poly", "entity_id"),
                          block.column("entity_poly", "pdbx_seq_one_letter_code_can")))  # fmt: skip
    seqs: dict[str, list[tuple[str, str]]] = {}
    seen: dict[str, set] = {}
    ps = block.table("entity_poly_seq")
    for e, num, mon in zip(ps.get("entity_id", []), ps.get("num", []), ps.get("mon_id", [])):
        if num in seen.setdefault(e, set()):  # hetero position: keep the first monomer
            continue
        seen[e].add(num)
        seqs.setdefault(e, []).append((num, mon))
    return kind, asym_entity, poly_type, {k: re.sub(r"\s+", "", v) for k, v in one_letter.items() if v not in MISSING}, seqs


def _component_bonds(block: CifBlock) -> dict[str, list[tuple[str, str, int]]]:
    t = block.table("chem_comp_bond")
    out: dict[str, list[tuple[str, str, int]]] = {}
    for comp, a, b, order in zip(t.get("comp_id", []), t.get("atom_id_1", []), t.get("atom_id_2", []),
                                 t.get("value_order", []) or itertools.repeat("SING")):  # fmt: skip
        out.setdefault(comp, []).append((a.strip('"'), b.strip('"'), _BOND_ORDER.get(order.upper()[:4], 1)))
    return out


def _distance_bonds(xyz: np.ndarray, elements: np.ndarray) -> list[tuple[int, int]]:
    """Bond guesses inside one component: distance below the sum of covalent radii plus 0.45 A."""
    if len(xyz) < 2:
        return []
    rad = np.array([_RADIUS.get(int(e), 1.3) for e in elements])
    d = np.linalg.norm(xyz[:, None] - xyz[None], axis=-1)
    i, j = np.nonzero(np.triu((d < rad[:, None] + rad[None] + 0.45) & (d > 0.4), 1))
    return list(zip(i.tolist(), j.tolist()))


def parse_mmcif(path: str, use_assembly: bool = True, assembly_id: str = "1", max_chains: int = 0,
                component_atoms: dict[str, set[str]] | None = None, drop_crystallization_aids: bool = False) -> tuple[Structure, Record]:  # fmt: skip
    """Read one entry. ``component_atoms`` (component -> allowed atom names) drops atoms a dictionary does not know.
    ``drop_crystallization_aids`` leaves out the non-polymer chains of an X-ray entry that consist of buffer or
    precipitant molecules only (``const.CRYSTALLIZATION_AIDS``; reference: data/prepare/structure.py:782).

    ``max_chains`` > 0 refuses assemblies that would expand to more chains (raises ``ValueError`` before any work).
    """
    block = read_cif(path)[0]
    stem = os.path.basename(str(path)).split(".")[0].lower()
    entry = (block.value("entry", "id") or block.name or stem).lower()
    name = stem if entry in ("model", "") else entry
    info = structure_info(block)
    kind, asym_entity, poly_type, one_letter, poly_seqs = _entities(block)
    observed = _atom_rows(block)
    comp_bonds = _component_bonds(block)

    plan = assembly_operations(block, assembly_id) if use_assembly else None
    if plan is None:
        plan = [(a, np.eye(4), True) for a in observed]
    plan = [p for p in plan if p[0] in observed]
    if max_chains and len(plan) > max_chains:
        raise ValueError(f"{len(plan)} chains > max {max_chains}")

    atoms, residues, chains, bonds, infos = [], [], [], [], []
    coords_of: dict[int, np.ndarray] = {}
    entity_of_key: dict[str, list[int]] = {}
    canonical: dict[int, str] = {}
    atom_index: dict[tuple[int, str, str], int] = {}  # (asym_id, residue key, atom name) -> atom row, for struct_conn
    copies: dict[str, int] = {}
    for label, mat, _ident in plan:
        src = observed[label]
        ent = asym_entity.get(label, "")
        mt = mol_type_of_polymer(poly_type[ent]) if ent in poly_type else const.MOL_NONPOLYMER
        if mt is None:
            continue
        if mt == const.MOL_NONPOLYMER:
            layout = [(k[0], src["res"][k]["comp"], k) for k in src["order"]]
            if drop_crystallization_aids and "X-RAY" in str(info.method or "").upper() and layout and all(
                    comp.strip().upper() in const.CRYSTALLIZATION_AIDS for _, comp, _ in layout):  # fmt: skip
                continue
        else:
            full = poly_seqs.get(ent)
            layout = [(num, mon, (num, "")) for num, mon in full] if full else [(k[0], src["res"][k]["comp"], k) for k in src["order"]]
        asym_id = len(chains)
        a0, r0 = len(atoms), len(residues)
        xyz_present = []
        for num, comp, key in layout:
            obs = src["res"].get(key)
            if obs is not None and obs["comp"] != comp:
                obs = None
            rtype, standard = residue_type(comp, mt) if mt != const.MOL_NONPOLYMER else (const.RES_TYPE_ORDER["UNK"], False)
            have = obs["atoms"] if obs else {}
            if comp in const.RESIDUE_ATOMS and mt != const.MOL_NONPOLYMER:
                names = list(const.RESIDUE_ATOMS[comp])
            else:
                names = [n for n in have if component_atoms is None or comp not in component_atoms or n in component_atoms[comp]]
            ra0 = len(atoms)
            for an in names:
                rec = have.get(an)
                if rec is None:
                    atoms.append((0.0, 0.0, 0.0, const.atom_element(an), 0.0, an[:4].encode(), False, 0.0))
                    continue
                p = mat[:3, :3] @ np.array(rec[1:4]) + mat[:3, 3]
                atoms.append((p[0], p[1], p[2], rec[4], rec[5], an[:4].encode(), True, rec[6]))
                xyz_present.append(p)
                atom_index[(asym_id, f"{key[0]}{key[1]}", an)] = len(atoms) - 1
            try:
                res_id = int(num)
            except ValueError:
                res_id = len(residues) - r0 + 1
            if len(atoms) == ra0 and mt == const.MOL_NONPOLYMER:
                continue
            residues.append((comp[:5].encode(), rtype, mt, res_id, ra0, len(atoms) - ra0, standard, bool(obs and have)))
            if comp not in const.RESIDUE_ATOMS or mt == const.MOL_NONPOLYMER:  # bonds inside a non-standard component
                local = {an: ra0 + k for k, an in enumerate(names) if an in have}
                if comp in comp_bonds:
                    bonds.extend((local[a], local[b], o) for a, b, o in comp_bonds[comp] if a in local and b in local)
                elif len(local) > 1:
                    idx = np.array(list(local.values()))
                    pts = np.array([[atoms[i][0], atoms[i][1], atoms[i][2]] for i in idx])
                    els = np.array([atoms[i][3] for i in idx])
                    bonds.extend((int(idx[i]), int(idx[j]), 1) for i, j in _distance_bonds(pts, els))
        if len(residues) == r0:
            del atoms[a0:]
            continue
        if mt != const.MOL_NONPOLYMER and ent in poly_seqs:
            seq_key = "|".join(PARENT.get(mon, mon) for _, mon in poly_seqs[ent])
            if ent in one_letter:
                canonical[asym_id] = one_letter[ent]
        else:
            seq_key = "|".join(PARENT.get(r[0].decode(), r[0].decode()) for r in residues[r0:])
        slot = entity_of_key.setdefault(seq_key, [len(entity_of_key), 0])
        entity_id, sym_id = slot[0], slot[1]
        slot[1] += 1
        k = copies.get(label, 0)
        copies[label] = k + 1
        cname = (label if k == 0 else f"{label}{k}")[:4]
        chains.append((cname.encode(), mt, entity_id, sym_id, asym_id, r0, len(residues) - r0, a0, len(atoms) - a0))
        coords_of[asym_id] = np.array(xyz_present, dtype=np.float64).reshape(-1, 3)
        h = sequence_hash(seq_key)
        infos.append(ChainInfo(asym_id, cname, mt, h, h, len(residues) - r0, entity_id, auth_chain_name=src["auth"],
                               res_name=residues[r0][0].decode() if mt == const.MOL_NONPOLYMER else None))  # fmt: skip
        chains[-1] = chains[-1] + (label,)  # remember the source label for struct_conn below

    label_to_asym: dict[str, list[int]] = {}
    for row in chains:
        label_to_asym.setdefault(row[-1], []).append(row[4])
    chains = [row[:-1] for row in chains]
    bonds.extend(_struct_conn_bonds(block, label_to_asym, atom_index))

    st = Structure(
        np.array(atoms, dtype=ATOM_DTYPE) if atoms else np.empty(0, ATOM_DTYPE),
        np.array(sorted(set(bonds)), dtype=BOND_DTYPE) if bonds else np.empty(0, BOND_DTYPE),
        np.array(residues, dtype=RESIDUE_DTYPE) if residues else np.empty(0, RESIDUE_DTYPE),
        np.array(chains, dtype=CHAIN_DTYPE) if chains else np.empty(0, CHAIN_DTYPE),
        name, canonical or None,
    )  # fmt: skip
    faces = find_interfaces(coords_of)
    info.num_chains, info.num_interfaces = len(chains), len(faces)
    return st, Record(name, infos, faces, info)


def _struct_conn_bonds(block: CifBlock, label_to_asym, atom_index) -> list[tuple[int, int, int]]:
    t = block.table("struct_conn")
    out = []
    for r in range(len(t.get("conn_type_id", []))):
        if not t["conn_type_id"][r].lower().startswith("covale"):
            continue
        ends = []
        for p in ("ptnr1", "ptnr2"):
            seq = t.get(f"{p}_label_seq_id", ["."])[r]
            if seq in MISSING:
                seq = t.get(f"{p}_auth_seq_id", ["."])[r]
            ins = t.get(f"pdbx_{p}_PDB_ins_code", ["."] * (r + 1))[r]
            ends.append((t[f"{p}_label_asym_id"][r], f"{seq}{'' if ins in MISSING else ins}", t[f"{p}_label_atom_id"][r].strip('"')))
        # the same symmetry copy of both ends (first copies pair with first copies)
        for a1, a2 in zip(label_to_asym.get(ends[0][0], []), label_to_asym.get(ends[1][0], [])):
            i, j = atom_index.get((a1, ends[0][1], ends[0][2])), atom_index.get((a2, ends[1][1], ends[1][2]))
            if i is not None and j is not None and i != j:
                out.append((min(i, j), max(i, j), 1))
    return out


def find_interfaces(coords_of: dict[int, np.ndarray], cutoff: float = INTERFACE_CUTOFF) -> list[InterfaceInfo]:
    """Chain pairs with any two resolved atoms closer than ``cutoff``."""
    from scipy.spatial import cKDTree

    ids = [c for c in sorted(coords_of) if len(coords_of[c])]
    trees = {c: cKDTree(coords_of[c]) for c in ids}
    boxes = {c: (coords_of[c].min(0) - cutoff, coords_of[c].max(0) + cutoff) for c in ids}
    out = []
    for a, b in itertools.combinations(ids, 2):
        if np.any(boxes[a][0] > boxes[b][1]) or np.any(boxes[b][0] > boxes[a][1]):
            continue
        if trees[a].count_neighbors(trees[b], cutoff) > 0:
            out.append(InterfaceInfo(a, b))
    return out
