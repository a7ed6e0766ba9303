"""Record-array containers of the data pipeline and their on-disk forms.

The field names, order and widths of the structured dtypes are a file format: ``.npz`` structures, MSAs and
manifest records written by the reference (data/types.py:20-109 for the dtypes, :111-297 ``Structure``,
:300-330 ``MSA``, :375-454 manifest records) load here unchanged and the other way round.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field

import numpy as np

from .io_cache import read_npz


def _dtype(spec: str) -> np.dtype:
    """``"x:f4 y:f4 name:S4"`` -> structured dtype (keeps the tables below one line each)."""
    return np.dtype([tuple(item.split(":")) for item in spec.split()])


ATOM_DTYPE = _dtype("x:f4 y:f4 z:f4 element:i1 charge:f2 name:S4 is_present:? b_factor:f4")
BOND_DTYPE = _dtype("atom_1:i4 atom_2:i4 type:i1")
RESIDUE_DTYPE = _dtype("name:S5 res_type:i2 mol_type:i1 res_id:i4 atom_idx:i4 atom_num:i2 is_standard:? is_present:?")
CHAIN_DTYPE = _dtype("name:S4 mol_type:i1 entity_id:i4 sym_id:i4 asym_id:i4 res_idx:i4 res_num:i4 atom_idx:i4 atom_num:i4")
TOKEN_DTYPE = _dtype(
    "token_idx:i4 residue_index:i4 res_type:i2 mol_type:i1 asym_id:i4 entity_id:i4 sym_id:i4 sym_token_index:i4 "
    "atom_idx:i4 atom_num:i2 center_x:f4 center_y:f4 center_z:f4 atom_in_res:i4"
)
TOKEN_BOND_DTYPE = _dtype("token_1:i4 token_2:i4 atom_1:i2 atom_2:i2")
_LEGACY_ATOM_DTYPE = np.dtype([d for d in ATOM_DTYPE.descr if d[0] != "b_factor"])  # files written before b_factor existed


def _plain(value):
    if isinstance(value, bytes):
        return value.decode("ascii", "replace")
    return value.item() if isinstance(value, np.generic) else value


def _rows_to_json(table: np.ndarray) -> list[dict]:
    return [{k: _plain(row[k]) for k in table.dtype.names} for row in table]


def _rows_from_json(rows: list[dict], dtype: np.dtype) -> np.ndarray:
    out = np.zeros(len(rows), dtype=dtype)
    for k in dtype.names:
        if rows:
            col = [r[k] for r in rows]
            out[k] = [c.encode("ascii") for c in col] if dtype[k].kind == "S" else col
    return out


@dataclass
class Structure:
    """Atoms, bonds, residues and chains of one entry as four record arrays (chains index residues index atoms)."""

    atoms: np.ndarray
    bonds: np.ndarray
    residues: np.ndarray
    chains: np.ndarray
    name: str = "unset"
    chain_canonical_seqs: dict[int, str] | None = None  # asym_id -> full one-letter sequence (incl. unresolved)

    # --- single-file form -------------------------------------------------------------------------------------
    def save(self, path) -> None:
        arrays = {"atoms": self.atoms, "bonds": self.bonds, "residues": self.residues, "chains": self.chains,
                  "name": np.array(self.name)}  # fmt: skip
        if self.chain_canonical_seqs:
            ids = sorted(self.chain_canonical_seqs)
            seqs = [self.chain_canonical_seqs[i] for i in ids]
            arrays["chain_canonical_asym_ids"] = np.asarray(ids, dtype=np.int32)
            arrays["chain_canonical_seqs"] = np.asarray(seqs, dtype=f"U{max(map(len, seqs))}")
        np.savez_compressed(str(path), **arrays)

    @classmethod
    def load(cls, path) -> "Structure":
        z = read_npz(str(path))
        atoms = z["atoms"]
        if atoms.dtype == ATOM_DTYPE:
            atoms = atoms.view(ATOM_DTYPE)
        else:
            old = atoms.view(_LEGACY_ATOM_DTYPE)
            atoms = np.zeros(len(old), dtype=ATOM_DTYPE)
            for k in old.dtype.names:
                atoms[k] = old[k]
        seqs = None
        if "chain_canonical_asym_ids" in z and "chain_canonical_seqs" in z:
            seqs = {int(i): str(s) for i, s in zip(z["chain_canonical_asym_ids"], z["chain_canonical_seqs"])}
        return cls(atoms, z["bonds"].view(BOND_DTYPE), z["residues"].view(RESIDUE_DTYPE), z["chains"].view(CHAIN_DTYPE),
                   str(z["name"]) if "name" in z else "unset", seqs)  # fmt: skip

    # --- split form: coordinates as arrays, everything else as JSON --------------------------------------------
    def save_split(self, directory) -> None:
        os.makedirs(directory, exist_ok=True)
        a = self.atoms
        np.savez_compressed(os.path.join(directory, "coords.npz"), x=a["x"], y=a["y"], z=a["z"], b_factor=a["b_factor"])
        meta = {
            "name": self.name,
            "chains": _rows_to_json(self.chains),
            "residues": _rows_to_json(self.residues),
            "bonds": _rows_to_json(self.bonds),
            "atoms": [{"element": int(r["element"]), "charge": float(r["charge"]), "name": _plain(r["name"]),
                       "is_present": bool(r["is_present"])} for r in a],  # fmt: skip
        }
        with open(os.path.join(directory, "meta.json"), "w") as f:
            json.dump(meta, f, indent=2)

    @classmethod
    def load_split(cls, directory) -> "Structure":
        xyz = read_npz(os.path.join(directory, "coords.npz"))
        with open(os.path.join(directory, "meta.json")) as f:
            meta = json.load(f)
        atoms = np.zeros(len(xyz["x"]), dtype=ATOM_DTYPE)
        for k in ("x", "y", "z", "b_factor"):
            atoms[k] = xyz[k]
        for k in ("element", "charge", "is_present"):
            if meta["atoms"]:
                atoms[k] = [r[k] for r in meta["atoms"]]
        if meta["atoms"]:
            atoms["name"] = [r["name"].encode("ascii") for r in meta["atoms"]]
        return cls(atoms, _rows_from_json(meta["bonds"], BOND_DTYPE), _rows_from_json(meta["residues"], RESIDUE_DTYPE),
                   _rows_from_json(meta["chains"], CHAIN_DTYPE), meta.get("name", "unset"))  # fmt: skip

    # --- helpers ----------------------------------------------------------------------------------------------
    def coords(self) -> np.ndarray:
        return np.stack([self.atoms["x"], self.atoms["y"], self.atoms["z"]], axis=-1)

    def chain_atoms(self, chain_row) -> slice:
        return slice(int(chain_row["atom_idx"]), int(chain_row["atom_idx"]) + int(chain_row["atom_num"]))

    def select_chains(self, keep_asym: list[int]) -> "Structure":
        """Sub-structure with the listed chains, indices rebuilt; bonds with a dropped end are removed."""
        keep = [c for c in self.chains if int(c["asym_id"]) in set(keep_asym)]
        new_atom = np.full(len(self.atoms), -1, dtype=np.int64)
        atoms, residues, chains = [], [], []
        a0 = r0 = 0
        for new_asym, c in enumerate(keep):
            res = self.residues[c["res_idx"] : c["res_idx"] + c["res_num"]].copy()
            sl = self.chain_atoms(c)
            new_atom[sl] = np.arange(a0, a0 + c["atom_num"])
            res["atom_idx"] += a0 - c["atom_idx"]
            row = c.copy()
            row["res_idx"], row["atom_idx"], row["asym_id"] = r0, a0, new_asym
            atoms.append(self.atoms[sl]), residues.append(res), chains.append(row)
            a0, r0 = a0 + int(c["atom_num"]), r0 + int(c["res_num"])
        bonds = self.bonds[(new_atom[self.bonds["atom_1"]] >= 0) & (new_atom[self.bonds["atom_2"]] >= 0)].copy()
        bonds["atom_1"], bonds["atom_2"] = new_atom[bonds["atom_1"]], new_atom[bonds["atom_2"]]
        seqs = None
        if self.chain_canonical_seqs:
            seqs = {i: self.chain_canonical_seqs[int(c["asym_id"])] for i, c in enumerate(keep)
                    if int(c["asym_id"]) in self.chain_canonical_seqs}  # fmt: skip
        cat = lambda parts, dt: np.concatenate(parts) if parts else np.empty(0, dtype=dt)  # noqa: E731
        return Structure(cat(atoms, ATOM_DTYPE), bonds, cat(residues, RESIDUE_DTYPE),
                         np.array(chains, dtype=CHAIN_DTYPE) if chains else np.empty(0, dtype=CHAIN_DTYPE), self.name, seqs)  # fmt: skip


@dataclass
class MSA:
    """Alignment of one chain: ``sequences`` int8 [S, N] (MSA vocabulary), ``mask`` bool, ``deletion_matrix`` int8."""

    sequences: np.ndarray
    mask: np.ndarray
    deletion_matrix: np.ndarray

    @property
    def is_empty(self) -> bool:
        return 0 in self.sequences.shape[:2]

    def save(self, path) -> None:
        np.savez_compressed(str(path), sequences=self.sequences, mask=self.mask, deletion_matrix=self.deletion_matrix)

    @classmethod
    def load(cls, path) -> "MSA":
        z = read_npz(str(path))
        return cls(z["sequences"], z["mask"], z["deletion_matrix"])

    @classmethod
    def empty(cls, length: int) -> "MSA":
        return cls(np.zeros((0, length), np.int8), np.zeros((0, length), bool), np.zeros((0, length), np.int8))


@dataclass
class ChainInfo:
    chain_id: int
    chain_name: str
    mol_type: int
    cluster_id: str | int
    msa_id: str | int
    num_residues: int
    entity_id: str | int | None = None
    paired_msa_id: str | int | None = None
    valid: bool = True
    auth_chain_name: str | None = None
    res_name: str | None = None


@dataclass
class InterfaceInfo:
    chain_1: int
    chain_2: int
    valid: bool = True


@dataclass
class StructureInfo:
    resolution: float | None = None
    method: str | None = None
    deposited: str | None = None
    released: str | None = None
    num_chains: int | None = None
    num_interfaces: int | None = None


@dataclass
class Record:
    """One manifest entry: which chains and interfaces an example has and where its files are keyed."""

    id: str
    chains: list[ChainInfo]
    interfaces: list[InterfaceInfo] = field(default_factory=list)
    structure_info: StructureInfo | None = None

    def to_dict(self) -> dict:
        optional = ("auth_chain_name", "res_name")
        chains = [{k: v for k, v in asdict(c).items() if not (k in optional and v is None)} for c in self.chains]
        out = {"id": self.id, "chains": chains, "interfaces": [asdict(i) for i in self.interfaces]}
        if self.structure_info is not None:
            out["structure_info"] = asdict(self.structure_info)
        return out

    @classmethod
    def from_dict(cls, d: dict) -> "Record":
        names = set(ChainInfo.__dataclass_fields__)
        chains = [ChainInfo(**{k: v for k, v in c.items() if k in names}) for c in d.get("chains", [])]
        faces = [InterfaceInfo(i["chain_1"], i["chain_2"], i.get("valid", True)) for i in d.get("interfaces", [])]
        si = d.get("structure_info")
        info = StructureInfo(**{k: v for k, v in si.items() if k in StructureInfo.__dataclass_fields__}) if si else None
        return cls(d["id"], chains, faces, info)


def load_manifest(path: str) -> list[Record]:
    with open(path) as f:
        return [Record.from_dict(d) for d in json.load(f)]


def save_manifest(records: list[Record], path: str) -> None:
    tmp = f"{path}.tmp"
    with open(tmp, "w") as f:
        json.dump([r.to_dict() for r in records], f)
    os.replace(tmp, path)
