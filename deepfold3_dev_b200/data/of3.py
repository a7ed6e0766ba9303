"""OpenFold 3 preprocessed data: structure import, columnar metadata cache and a reader for training.

Reference: data/prepare/openfold3.py:88-453 (atom-array conversion), data/prepare/of3_pdb_cache.py (columnar cache),
data/module/of3_dataset.py and of3_pdb_dataset.py (datasets over OpenFold 3 directories). The OpenFold 3 files are a
data format here, nothing of that project is used:

* structures are ``.npz`` files with flat per-atom arrays ``coord [n, 3]``, ``chain_id``, ``res_id``, ``res_name``,
  ``atom_name``, ``element`` and optionally ``ins_code``, ``molecule_type_id`` (0 protein, 1 RNA, 2 DNA, 3 ligand),
  ``occupancy``, ``charge``, ``entity_id`` / ``label_entity_id``, ``label_asym_id`` / ``auth_asym_id`` and ``bonds``
  ``[m, 3]`` (atom, atom, type);
* the dataset cache is one JSON ``{"structure_data": {pdb id: {"release_date", "resolution", "experimental_method",
  "chains": {chain id: {"cluster_id", "molecule_type", "alignment_representative_id", "template_ids", ...}}}}}``.
"""

from __future__ import annotations

import json
import os

import numpy as np

from . import const, io_cache, paths
from .io_cache import read_npz
from .parse.mmcif import _element, find_interfaces, residue_type, sequence_hash
from .types import ATOM_DTYPE, BOND_DTYPE, CHAIN_DTYPE, RESIDUE_DTYPE, ChainInfo, Record, Structure, StructureInfo, save_manifest

OF3_MOL_TYPE = {0: const.MOL_PROTEIN, 1: const.MOL_RNA, 2: const.MOL_DNA, 3: const.MOL_NONPOLYMER}
_MOL_BY_NAME = {"PROTEIN": const.MOL_PROTEIN, "RNA": const.MOL_RNA, "DNA": const.MOL_DNA, "LIGAND": const.MOL_NONPOLYMER}
_ONE_LETTER = {i: (const.RES_TYPE_INDEX_TO_NAME[i] if 22 <= i <= 25 else const.RES_TYPE_INDEX_TO_NAME[i][1:] if 26 <= i <= 29 else "N")
               for i in range(22, 31)}  # fmt: skip


def _text(arr) -> np.ndarray:
    arr = np.asarray(arr)
    return np.char.decode(arr, "ascii") if arr.dtype.kind == "S" else arr.astype(str)


def _runs(*keys) -> np.ndarray:
    """Start index of every run of equal key tuples."""
    n = len(keys[0])
    change = np.zeros(n, dtype=bool)
    change[0] = True
    for k in keys:
        change[1:] |= k[1:] != k[:-1]
    return np.flatnonzero(change)


def _letters(res_types: np.ndarray, mol_type: int) -> str:
    if mol_type == const.MOL_PROTEIN:
        one = {v: const.PROTEIN_1[k] for k, v in const.RES_TYPE_ORDER.items() if v < 20} if hasattr(const, "PROTEIN_1") else {}
        names = [const.RES_TYPE_INDEX_TO_NAME.get(int(t), "UNK") for t in res_types]
        return "".join(one.get(int(t), _three_to_one(n)) for t, n in zip(res_types, names))
    return "".join(_ONE_LETTER.get(int(t), "N") for t in res_types)


def _three_to_one(name: str) -> str:
    table = {"ALA": "A", "ARG": "R", "ASN": "N", "ASP": "D", "CYS": "C", "GLN": "Q", "GLU": "E", "GLY": "G", "HIS": "H",
             "ILE": "I", "LEU": "L", "LYS": "K", "MET": "M", "PHE": "F", "PRO": "P", "SER": "S", "THR": "T", "TRP": "W",
             "TYR": "Y", "VAL": "V"}  # fmt: skip
    return table.get(name, "X")


def convert_atom_array(data, name: str) -> tuple[Structure, Record]:
    """One OpenFold 3 atom array -> ``Structure`` plus its manifest ``Record`` (chains in file order)."""
    coord = np.asarray(data["coord"], dtype=np.float32).reshape(-1, 3)
    n = len(coord)
    if n == 0:
        raise ValueError("empty atom array")
    chain_key, res_id = _text(data["chain_id"]), np.asarray(data["res_id"]).astype(np.int64)
    res_name, atom_name, element = _text(data["res_name"]), _text(data["atom_name"]), _text(data["element"])
    ins = _text(data["ins_code"]) if "ins_code" in data else np.full(n, "", dtype="<U1")
    of3_mol = np.asarray(data["molecule_type_id"]).astype(np.int64) if "molecule_type_id" in data else None
    occupancy = np.asarray(data["occupancy"], dtype=np.float32) if "occupancy" in data else np.ones(n, np.float32)
    charge = np.asarray(data["charge"], dtype=np.float32) if "charge" in data else np.zeros(n, np.float32)
    entity = None
    for key in ("entity_id", "label_entity_id"):
        if key in data:
            entity = np.asarray(data[key]).astype(np.int64)
            break
    present = np.isfinite(coord).all(axis=1) & (occupancy > 0)
    coord = np.where(present[:, None], coord, 0.0)

    atoms = np.zeros(n, dtype=ATOM_DTYPE)
    atoms["x"], atoms["y"], atoms["z"] = coord[:, 0], coord[:, 1], coord[:, 2]
    atoms["element"] = [_element(e, a) for e, a in zip(element, atom_name)]
    atoms["charge"] = charge.astype(np.float16)
    atoms["name"] = [a[:4].encode("ascii", "replace") for a in atom_name]
    atoms["is_present"] = present

    chain_starts = _runs(chain_key)
    res_starts = _runs(chain_key, res_id, ins, res_name)
    res_counts = np.diff(np.append(res_starts, n))
    res_chain = np.searchsorted(chain_starts, res_starts, side="right") - 1
    chain_mol = []
    for ci, a0 in enumerate(chain_starts):
        if of3_mol is not None:
            chain_mol.append(OF3_MOL_TYPE.get(int(of3_mol[a0]), const.MOL_NONPOLYMER))
        else:  # no type column: a chain whose first residue is a standard amino acid / nucleotide is a polymer of that kind
            first = res_name[a0]
            chain_mol.append(const.MOL_PROTEIN if first in const.RES_TYPE_ORDER and const.RES_TYPE_ORDER[first] < 21
                             else const.MOL_RNA if first in ("A", "G", "C", "U") else const.MOL_DNA if first in ("DA", "DG", "DC", "DT")
                             else const.MOL_NONPOLYMER)  # fmt: skip
    residues = np.zeros(len(res_starts), dtype=RESIDUE_DTYPE)
    for ri, a0 in enumerate(res_starts):
        mt = chain_mol[res_chain[ri]]
        rtype, standard = residue_type(res_name[a0], mt)
        sl = slice(a0, a0 + res_counts[ri])
        residues[ri] = (res_name[a0][:5].encode("ascii", "replace"), rtype, mt, int(res_id[a0]), a0, res_counts[ri], standard,
                        bool(present[sl].any()))  # fmt: skip

    chains = np.zeros(len(chain_starts), dtype=CHAIN_DTYPE)
    infos, coords_of, seqs = [], {}, {}
    chain_res_start = np.searchsorted(res_starts, chain_starts)
    chain_res_count = np.diff(np.append(chain_res_start, len(res_starts)))
    chain_atom_count = np.diff(np.append(chain_starts, n))
    entity_of_key: dict[str, list[int]] = {}
    for ci, a0 in enumerate(chain_starts):
        r0, rn = int(chain_res_start[ci]), int(chain_res_count[ci])
        mt = chain_mol[ci]
        key = "|".join(residues["name"][r0 : r0 + rn].astype(str))
        slot = entity_of_key.setdefault(f"{mt}:{key}" if entity is None else f"e{int(entity[a0])}", [len(entity_of_key), 0])
        sym_id, slot[1] = slot[1], slot[1] + 1
        label = str(chain_key[a0])[:4]
        chains[ci] = (label.encode("ascii", "replace"), mt, slot[0], sym_id, ci, r0, rn, a0, chain_atom_count[ci])
        sl = slice(a0, a0 + chain_atom_count[ci])
        coords_of[ci] = coord[sl][present[sl]].astype(np.float64)
        h = sequence_hash(key)
        if mt != const.MOL_NONPOLYMER:
            seqs[ci] = _letters(residues["res_type"][r0 : r0 + rn], mt)
        infos.append(ChainInfo(ci, label, mt, h, h, rn, slot[0],
                               res_name=str(residues["name"][r0].astype(str)) if mt == const.MOL_NONPOLYMER else None))  # fmt: skip

    bonds = np.zeros(0, dtype=BOND_DTYPE)
    if "bonds" in data and len(data["bonds"]):
        raw = np.asarray(data["bonds"]).astype(np.int64).reshape(-1, 3)
        raw = raw[(raw[:, 0] < n) & (raw[:, 1] < n)]
        # keep what the model reads as token bonds: every bond with an end outside the standard polymer residues
        res_of_atom = np.repeat(np.arange(len(res_starts)), res_counts)
        std = residues["is_standard"][res_of_atom]
        raw = raw[~(std[raw[:, 0]] & std[raw[:, 1]]) | (res_of_atom[raw[:, 0]] != res_of_atom[raw[:, 1]])]
        bonds = np.zeros(len(raw), dtype=BOND_DTYPE)
        bonds["atom_1"], bonds["atom_2"], bonds["type"] = raw[:, 0], raw[:, 1], np.clip(raw[:, 2], 0, 127)
    st = Structure(atoms, bonds, residues, chains, name, seqs or None)
    rec = Record(name, infos, find_interfaces(coords_of), StructureInfo(num_chains=len(infos)))
    rec.structure_info.num_interfaces = len(rec.interfaces)
    return st, rec


def load_dataset_cache(path: str) -> dict[str, dict]:
    with open(path) as f:
        raw = json.load(f)
    entries = raw.get("structure_data", raw)
    return {str(k).lower(): v for k, v in entries.items() if isinstance(v, dict)}


def scan_structures(root: str) -> list[tuple[str, str]]:
    """``(id, path)`` of every structure file: ``<root>/<id>/<id>.npz`` or flat ``<root>/<id>.npz``."""
    found = []
    for entry in sorted(os.listdir(root)):
        full = os.path.join(root, entry)
        if os.path.isdir(full):
            for cand in (os.path.join(full, f"{entry}.npz"), *sorted(p for p in (os.path.join(full, f) for f in os.listdir(full)) if p.endswith(".npz"))):
                if os.path.exists(cand):
                    found.append((entry.lower(), cand))
                    break
        elif entry.endswith(".npz"):
            found.append((entry[:-4].lower(), full))
    return found


def apply_cache_entry(rec: Record, entry: dict | None) -> None:
    """Resolution, method, release date and per-chain cluster ids of the dataset cache, where it has them."""
    if not entry:
        return
    info = rec.structure_info or StructureInfo()
    info.resolution = entry.get("resolution", info.resolution)
    info.method = entry.get("experimental_method", info.method)
    info.released = entry.get("release_date", info.released)
    rec.structure_info = info
    chains = entry.get("chains") or {}
    for c in rec.chains:
        meta = chains.get(c.chain_name) or chains.get(str(c.chain_id))
        if meta and meta.get("cluster_id") not in (None, ""):
            c.cluster_id = str(meta["cluster_id"])


def convert_directory(of3_dir: str, out_dir: str, cache_path: str | None = None, limit: int | None = None) -> tuple[int, int]:
    cache = load_dataset_cache(cache_path) if cache_path else {}
    os.makedirs(os.path.join(out_dir, "structures"), exist_ok=True)
    records, skipped = [], 0
    for pdb_id, path in scan_structures(of3_dir)[: limit or None]:
        try:
            st, rec = convert_atom_array(read_npz(path), pdb_id)
        except (KeyError, ValueError) as exc:
            skipped += 1
            print(f"skipping {path}: {exc}")
            continue
        apply_cache_entry(rec, cache.get(pdb_id))
        st.save(paths.structure(out_dir, pdb_id))
        records.append(rec)
    save_manifest(records, paths.manifest(out_dir))
    return len(records), skipped


# ---------------------------------------------------------------------------------------------------------------------------
# Columnar cache: the JSON parsed once into flat arrays that every rank and loader worker memory-maps.
_ENTRY_COLUMNS = ("entry_id", "release_date", "resolution", "method", "chain_start", "chain_count")
_CHAIN_COLUMNS = ("chain_name", "mol_type", "cluster_id", "msa_representative", "template_start", "template_count")


def build_columnar_cache(cache_file: str, out_dir: str, with_templates: bool = True) -> tuple[int, int]:
    cache = load_dataset_cache(cache_file)
    os.makedirs(out_dir, exist_ok=True)
    ids = sorted(cache)
    e_date, e_res, e_method, e_start, e_count = [], [], [], [], []
    c_name, c_mol, c_cluster, c_rep, t_start, t_count, templates = [], [], [], [], [], [], []
    for pdb_id in ids:
        entry = cache[pdb_id]
        chains = entry.get("chains") or {}
        e_date.append(str(entry.get("release_date") or ""))
        e_res.append(float(entry.get("resolution") or 0.0))
        e_method.append(str(entry.get("experimental_method") or ""))
        e_start.append(len(c_name))
        e_count.append(len(chains))
        for cname, meta in chains.items():
            c_name.append(str(cname))
            c_mol.append(_MOL_BY_NAME.get(str(meta.get("molecule_type", "")).upper(), -1))
            c_cluster.append(str(meta.get("cluster_id") or ""))
            c_rep.append(str(meta.get("alignment_representative_id") or ""))
            ids_t = list(meta.get("template_ids") or []) if with_templates else []
            t_start.append(len(templates))
            t_count.append(len(ids_t))
            templates.extend(str(t) for t in ids_t)

    def text(values):
        return np.asarray(values, dtype=f"S{max(1, max((len(v) for v in values), default=1))}")

    columns = {
        "entry_id": text(ids), "release_date": text(e_date), "resolution": np.asarray(e_res, np.float32), "method": text(e_method),
        "chain_start": np.asarray(e_start, np.int64), "chain_count": np.asarray(e_count, np.int32), "chain_name": text(c_name),
        "mol_type": np.asarray(c_mol, np.int8), "cluster_id": text(c_cluster), "msa_representative": text(c_rep),
        "template_start": np.asarray(t_start, np.int64), "template_count": np.asarray(t_count, np.int32),
        "template_id": text(templates),
    }  # fmt: skip
    for name, col in columns.items():
        np.save(os.path.join(out_dir, f"{name}.npy"), col)
    with open(os.path.join(out_dir, "meta.json"), "w") as f:
        json.dump({"entries": len(ids), "chains": len(c_name), "templates": len(templates), "columns": sorted(columns)}, f)
    return len(ids), len(c_name)


class ColumnarCache:
    """Read side of ``build_columnar_cache``: columns are memory-mapped, rows are looked up by binary search on the id."""

    def __init__(self, root: str):
        with open(os.path.join(root, "meta.json")) as f:
            self.meta = json.load(f)
        self.col = {name: np.load(os.path.join(root, f"{name}.npy"), mmap_mode="r") for name in self.meta["columns"]}

    def __len__(self) -> int:
        return int(self.meta["entries"])

    def index_of(self, entry_id: str) -> int:
        ids = self.col["entry_id"]
        key = entry_id.lower().encode()
        i = int(np.searchsorted(ids, key))
        return i if i < len(ids) and ids[i] == key else -1

    def entry(self, i: int) -> dict:
        c = self.col
        s, n = int(c["chain_start"][i]), int(c["chain_count"][i])
        chains = []
        for k in range(s, s + n):
            t0, tn = int(c["template_start"][k]), int(c["template_count"][k])
            chains.append({"chain_name": c["chain_name"][k].decode(), "mol_type": int(c["mol_type"][k]),
                           "cluster_id": c["cluster_id"][k].decode(), "msa_representative": c["msa_representative"][k].decode(),
                           "template_ids": [t.decode() for t in c["template_id"][t0 : t0 + tn]]})  # fmt: skip
        return {"id": c["entry_id"][i].decode(), "release_date": c["release_date"][i].decode(),
                "resolution": float(c["resolution"][i]), "method": c["method"][i].decode(), "chains": chains}  # fmt: skip

    def select(self, max_release_date: str | None = None, max_resolution: float | None = None) -> np.ndarray:
        """Indices of entries released on or before the date (ISO strings compare in order) within the resolution."""
        keep = np.ones(len(self), dtype=bool)
        if max_release_date:
            dates = np.asarray(self.col["release_date"])
            keep &= (dates != b"") & (dates <= max_release_date.encode())
        if max_resolution:
            res = np.asarray(self.col["resolution"])
            keep &= (res > 0) & (res <= max_resolution)
        return np.flatnonzero(keep)

    def cluster_weights(self, indices: np.ndarray) -> np.ndarray:
        """Sampling weight per entry: the sum over its chains of 1 / (size of the chain's cluster among ``indices``)."""
        c = self.col
        counts: dict[bytes, int] = {}
        for i in indices:
            s, n = int(c["chain_start"][i]), int(c["chain_count"][i])
            for cid in c["cluster_id"][s : s + n]:
                counts[bytes(cid)] = counts.get(bytes(cid), 0) + 1
        out = np.zeros(len(indices), dtype=np.float64)
        for k, i in enumerate(indices):
            s, n = int(c["chain_start"][i]), int(c["chain_count"][i])
            out[k] = sum(1.0 / counts[bytes(cid)] for cid in c["cluster_id"][s : s + n]) if n else 0.0
        return out


class OF3StructureDataset:
    """Map-style dataset straight over an OpenFold 3 structure directory (no import step): each item is converted on
    the fly, cropped and featurised like a prepared example. ``cache_dir`` (a ``ColumnarCache``) supplies release-date
    and resolution filters and cluster-balanced sampling weights; alignments are looked up under ``msa_dir`` by the
    chains' sequence hashes and missing ones fall back to the single sequence."""

    def __init__(self, of3_dir: str, cache_dir: str | None = None, msa_dir: str | None = None, max_tokens: int = 384,
                 max_atoms: int = 4096, max_msa_rows: int = 1024, max_release_date: str | None = None,
                 max_resolution: float | None = None, seed: int = 0, crop_weights: dict | None = None,
                 is_distillation: bool = False, atomize_prob: float = 0.0, atomize_source: str = "random",
                 atomize_max_residues: int = 0):  # fmt: skip
        self.atomize = {"atomize_prob": atomize_prob, "atomize_source": atomize_source, "atomize_max_residues": atomize_max_residues}
        structures = os.path.join(of3_dir, "structures")
        self.items = scan_structures(structures if os.path.isdir(structures) else of3_dir)
        self.cache = ColumnarCache(cache_dir) if cache_dir else None
        self._weights = None
        if self.cache is not None:
            allowed = {self.cache.col["entry_id"][i].decode() for i in self.cache.select(max_release_date, max_resolution)}
            self.items = [it for it in self.items if it[0] in allowed]
            idx = np.asarray([self.cache.index_of(pid) for pid, _ in self.items], dtype=np.int64)
            self._weights = self.cache.cluster_weights(idx)
        from . import pack as packs

        packs.register(of3_dir)  # alignments may live in {of3_dir}/_pack
        if msa_dir is None and io_cache.exists(os.path.join(of3_dir, "msa")):
            msa_dir = os.path.join(of3_dir, "msa")
        self.msa_dir, self.max_tokens, self.max_atoms, self.max_msa_rows, self.seed = msa_dir, max_tokens, max_atoms, max_msa_rows, seed
        self.crop_weights, self.is_distillation = crop_weights, is_distillation
        self.msa_read = self.msa_skipped = 0

    def weights(self) -> list[float]:
        """Sampling weights: cluster-balanced when the metadata cache is there, uniform otherwise."""
        return [1.0] * len(self.items) if self._weights is None else [float(w) for w in self._weights]

    def __len__(self) -> int:
        return len(self.items)

    def __getitem__(self, index: int) -> dict:
        from .datasets import featurize_record

        pdb_id, path = self.items[index]
        st, rec = convert_atom_array(read_npz(path), pdb_id)
        if self.cache is not None:
            i = self.cache.index_of(pdb_id)
            if i >= 0:
                e = self.cache.entry(i)
                apply_cache_entry(rec, {"resolution": e["resolution"], "experimental_method": e["method"], "release_date": e["release_date"],
                                        "chains": {c["chain_name"]: c for c in e["chains"]}})  # fmt: skip
        feats, read, skipped = featurize_record(st, rec, self._msa, max_tokens=self.max_tokens, max_atoms=self.max_atoms,
                                                crop_weights=self.crop_weights, max_msa_rows=self.max_msa_rows,
                                                seed=self.seed * 7_654_321 + index, is_distillation=self.is_distillation,
                                                **self.atomize)  # fmt: skip
        self.msa_read, self.msa_skipped = self.msa_read + read, self.msa_skipped + skipped
        return feats

    def _msa(self, chain):
        """The alignment stored for a chain's sequence hash under ``msa_dir`` (``.npz`` or ``.a3m``), if any."""
        from .parse.a3m import msa_from_a3m_file
        from .types import MSA

        if not self.msa_dir:
            return None
        base = os.path.join(self.msa_dir, str(chain.msa_id))
        if io_cache.exists(base + ".npz"):
            return MSA.load(base + ".npz")
        if io_cache.exists(base + ".a3m"):
            return msa_from_a3m_file(base + ".a3m", chain.mol_type, self.max_msa_rows)
        return None
