"""mmCIF output of predicted structures.

One ``data_`` block with ``_entry``, ``_struct``, ``_entity`` / ``_entity_poly``, ``_struct_asym``, the
per-residue pLDDT table (``_ma_qa_metric_local``) and ``_atom_site`` with the pLDDT in the B-factor column;
several samples become several ``pdbx_PDB_model_num`` values (reference: io/mmcif.py:106-379). Written
directly as text: no structure library is needed.
"""

from __future__ import annotations

import os
from collections.abc import Sequence

import torch

from ..data import const

ELEMENT_SYMBOLS = (
    "X H He Li Be B C N O F Ne Na Mg Al Si P S Cl Ar K Ca Sc Ti V Cr Mn Fe Co Ni Cu Zn Ga Ge As Se Br Kr Rb Sr Y Zr Nb Mo "
    "Tc Ru Rh Pd Ag Cd In Sn Sb Te I Xe Cs Ba La Ce Pr Nd Pm Sm Eu Gd Tb Dy Ho Er Tm Yb Lu Hf Ta W Re Os Ir Pt Au Hg Tl "
    "Pb Bi Po At Rn Fr Ra Ac Th Pa U Np Pu Am Cm Bk Cf Es Fm Md No Lr Rf Db Sg Bh Hs Mt Ds Rg Cn Nh Fl Mc Lv Ts Og"
).split()


def asym_id_to_chain_name(asym_id: int) -> str:
    """0 -> A, 25 -> Z, 26 -> AA, ... (spreadsheet-column numbering)."""
    n, out = int(asym_id), ""
    while True:
        out = chr(ord("A") + n % 26) + out
        n = n // 26 - 1
        if n < 0:
            return out


def resolve_chain_name(asym_id: int, chain_names: Sequence[str | None] | None = None) -> str:
    if chain_names is not None and asym_id < len(chain_names) and chain_names[asym_id]:
        return str(chain_names[asym_id])
    return asym_id_to_chain_name(asym_id)


def decode_atom_name(chars) -> str:
    """Four codes (ASCII - 32, 0 = blank) back to the atom name."""
    return "".join(chr(int(c) + 32) for c in chars if int(c) > 0).strip()


def _quote(v: str) -> str:
    v = str(v)
    if v == "":
        return "."
    if any(c in v for c in " '\"#") or v[0] in "_;$[]":
        return f'"{v}"' if '"' not in v else f"'{v}'"
    return v


def _entity_type(mol_type: int) -> tuple[str, str]:
    return {const.MOL_PROTEIN: ("polymer", "polypeptide(L)"), const.MOL_DNA: ("polymer", "polydeoxyribonucleotide"),
            const.MOL_RNA: ("polymer", "polyribonucleotide")}.get(int(mol_type), ("non-polymer", ""))  # fmt: skip


def structure_to_mmcif(positions, plddt_atoms, features: dict, entry_id: str = "prediction", title: str | None = None,
                       chain_names: Sequence[str | None] | None = None, res_names: Sequence[str] | None = None) -> str:  # fmt: skip
    """``positions`` ``[S, N, M, 3]`` (or ``[N, M, 3]``), ``plddt_atoms`` same without the last axis or ``None``."""
    pos = positions if positions.dim() == 4 else positions[None]
    pos = pos.detach().float().cpu()
    S, N, M, _ = pos.shape
    bf = None if plddt_atoms is None else (plddt_atoms if plddt_atoms.dim() == 3 else plddt_atoms[None]).detach().float().cpu()
    f = {k: v.detach().cpu() for k, v in features.items() if isinstance(v, torch.Tensor)}
    mask = f["ref_mask"].bool() & f["seq_mask"].bool()[:, None]
    asym, res_idx, mol = f["asym_id"].tolist(), f["residue_index"].tolist(), f["mol_type"].tolist()
    rtype = f["res_type"].tolist()
    names3 = list(res_names) if res_names is not None else [const.RES_TYPE_INDEX_TO_NAME.get(t, "UNK") for t in rtype]
    names3 = ["LIG" if (mol[i] == const.MOL_NONPOLYMER and names3[i] in ("UNK", "-")) else names3[i] for i in range(N)]
    ent = f["entity_id"].tolist() if "entity_id" in f else asym
    out = [f"data_{entry_id}", "#", f"_entry.id {entry_id}", "#"]
    if title:
        out += [f"_struct.entry_id {entry_id}", f"_struct.title {_quote(title)}", "#"]
    # entities
    ents: dict[int, int] = {}
    for i in range(N):
        if mask[i].any():
            ents.setdefault(ent[i], mol[i])
    out += ["loop_", "_entity.id", "_entity.type", "_entity.pdbx_description"]
    out += [f"{e + 1} {_entity_type(mt)[0]} ." for e, mt in ents.items()]
    out += ["#", "loop_", "_entity_poly.entity_id", "_entity_poly.type"]
    out += [f"{e + 1} {_quote(_entity_type(mt)[1])}" for e, mt in ents.items() if _entity_type(mt)[0] == "polymer"] or ["? ?"]
    chains: dict[int, int] = {}
    for i in range(N):
        if mask[i].any():
            chains.setdefault(asym[i], ent[i])
    out += ["#", "loop_", "_struct_asym.id", "_struct_asym.entity_id"]
    out += [f"{resolve_chain_name(a, chain_names)} {e + 1}" for a, e in chains.items()]
    if bf is not None:  # per-residue pLDDT of the first model
        out += ["#", "loop_", "_ma_qa_metric_local.ordinal_id", "_ma_qa_metric_local.model_id",
                "_ma_qa_metric_local.label_asym_id", "_ma_qa_metric_local.label_seq_id",
                "_ma_qa_metric_local.label_comp_id", "_ma_qa_metric_local.metric_id", "_ma_qa_metric_local.metric_value"]  # fmt: skip
        k, seen = 0, set()
        for i in range(N):
            key = (asym[i], res_idx[i])
            if not mask[i].any() or key in seen:
                continue
            seen.add(key)
            same = [j for j in range(i, N) if (asym[j], res_idx[j]) == key]
            vals = torch.cat([bf[0, j][mask[j]] for j in same])
            k += 1
            out.append(f"{k} 1 {resolve_chain_name(asym[i], chain_names)} {res_idx[i] + 1} {names3[i]} 1 {vals.mean():.2f}")
    out += ["#", "loop_"] + [f"_atom_site.{c}" for c in (
        "group_PDB", "id", "type_symbol", "label_atom_id", "label_alt_id", "label_comp_id", "label_asym_id",
        "label_entity_id", "label_seq_id", "pdbx_PDB_ins_code", "Cartn_x", "Cartn_y", "Cartn_z", "occupancy",
        "B_iso_or_equiv", "auth_seq_id", "auth_asym_id", "pdbx_PDB_model_num")]  # fmt: skip
    chars = f["ref_atom_name_chars"]
    elem = f["ref_element"].tolist()
    for s in range(S):
        serial = 0
        for i in range(N):
            group = "HETATM" if mol[i] == const.MOL_NONPOLYMER else "ATOM"
            ch = resolve_chain_name(asym[i], chain_names)
            for a in range(M):
                if not mask[i, a]:
                    continue
                serial += 1
                e = elem[i][a]
                sym = ELEMENT_SYMBOLS[e] if 0 <= e < len(ELEMENT_SYMBOLS) else "X"
                x, y, z = pos[s, i, a].tolist()
                b = float(bf[s, i, a]) if bf is not None else 0.0
                out.append(f"{group} {serial} {sym.upper()} {_quote(decode_atom_name(chars[i, a]) or sym)} . {names3[i]} {ch} "
                           f"{ent[i] + 1} {res_idx[i] + 1} ? {x:.3f} {y:.3f} {z:.3f} 1.00 {b:.2f} {res_idx[i] + 1} {ch} {s + 1}")  # fmt: skip
    out.append("#")
    return "\n".join(out) + "\n"


def save_mmcif(path: str, output, features: dict, num_plddt_bins: int = 50, title: str | None = None,
               sample_idx: int | None = None, chain_names: Sequence[str | None] | None = None) -> None:  # fmt: skip
    """Write ``output.atom_positions`` (all samples as models, or one ``sample_idx``) with pLDDT B-factors."""
    from .confidences import compute_plddt

    pos = output.atom_positions
    per_atom = None
    if getattr(output, "plddt", None) is not None:
        per_atom, _ = compute_plddt(output.plddt.float().cpu(), features["ref_mask"].float().cpu(), num_plddt_bins)
    if sample_idx is not None:
        pos = pos[sample_idx : sample_idx + 1]
        per_atom = None if per_atom is None else per_atom[sample_idx : sample_idx + 1]
    text = structure_to_mmcif(pos, per_atom, features, entry_id=os.path.splitext(os.path.basename(path))[0] or "prediction",
                              title=title, chain_names=chain_names)  # fmt: skip
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with open(path, "w") as fh:
        fh.write(text)
