"""Job descriptions in four JSON dialects -> ``JobInput`` (reference: data/parse/json_input.py:56-803).

* ``alphafold3``: ``{"name", "modelSeeds", "sequences": [{"protein"|"rna"|"dna"|"ligand": {"id", ...}}]}``
* ``alphafoldserver``: a list of jobs with ``proteinChain`` / ``rnaSequence`` / ``dnaSequence`` / ``ligand`` /
  ``ion`` entries carrying ``count``
* ``protenix``: ``[{"name", "sequences": [{"proteinChain": {"sequence", "count", "msa": {...}}}, ...]}]``
* ``deepfold3``: the union of the key styles above

The dialect is taken from a ``"dialect"`` field or detected from the keys. MSAs may be inline A3M text
or paths relative to the JSON file. MSA search services are a separate process boundary and are not
called from here: a chain without an MSA gets a single-row alignment (its own sequence).
"""

from __future__ import annotations

import dataclasses
import json
import os

from .. import const


@dataclasses.dataclass
class ProteinChainInput:
    ids: list[str]
    sequence: str
    unpaired_msa: str | None = None  # A3M text
    paired_msa: str | None = None
    modifications: list[tuple[str, int]] = dataclasses.field(default_factory=list)  # (CCD code, 1-based position)
    templates: list[dict] = dataclasses.field(default_factory=list)
    mol_type: int = const.MOL_PROTEIN


@dataclasses.dataclass
class NucleotideChainInput:
    ids: list[str]
    sequence: str
    mol_type: int = const.MOL_RNA
    unpaired_msa: str | None = None
    modifications: list[tuple[str, int]] = dataclasses.field(default_factory=list)


@dataclasses.dataclass
class LigandChainInput:
    ids: list[str]
    ccd_codes: list[str] = dataclasses.field(default_factory=list)
    smiles: str | None = None
    mol_type: int = const.MOL_NONPOLYMER


@dataclasses.dataclass
class BondedAtomPair:
    a: tuple[str, int, str]  # (chain id, 1-based residue, atom name)
    b: tuple[str, int, str]


@dataclasses.dataclass
class JobInput:
    name: str
    chains: list
    seeds: list[int] = dataclasses.field(default_factory=lambda: [0])
    bonded_atom_pairs: list[BondedAtomPair] = dataclasses.field(default_factory=list)
    dialect: str = "deepfold3"
    user_ccd: str | None = None

    @property
    def num_chains(self) -> int:
        return sum(len(c.ids) for c in self.chains)


def _ids(raw) -> list[str]:
    return [raw] if isinstance(raw, str) else list(raw)


def _letters(n: int, start: int) -> list[str]:
    from ...io.mmcif import asym_id_to_chain_name

    return [asym_id_to_chain_name(start + i) for i in range(n)]


def _read_text(base_dir: str, path: str | None, inline: str | None) -> str | None:
    if inline:
        return inline
    if path:
        p = path if os.path.isabs(path) else os.path.join(base_dir, path)
        with open(p) as f:
            return f.read()
    return None


def _mods(raw, code_key, pos_key) -> list[tuple[str, int]]:
    return [(str(m[code_key]).replace("CCD_", ""), int(m[pos_key])) for m in (raw or [])]


def detect_dialect(entry: dict) -> str:
    if isinstance(entry.get("dialect"), str):
        return entry["dialect"].lower()
    keys = set()
    for s in entry.get("sequences", []):
        keys.update(s.keys())
    if keys & {"protein", "rna", "dna"}:
        return "alphafold3"
    if keys & {"proteinChain", "rnaSequence", "dnaSequence"}:
        has_msa = any("msa" in v or "templatesPath" in v for s in entry.get("sequences", []) for v in s.values() if isinstance(v, dict))
        return "protenix" if has_msa else "alphafoldserver"
    return "deepfold3"


def _templates(spec: dict, base_dir: str) -> list[dict]:
    """Inline ``templates`` or the hit list behind ``templatesPath``; every hit remembers where relative paths start."""
    hits, root = list(spec.get("templates") or []), base_dir
    path = spec.get("templatesPath")
    if not hits and path:
        full = path if os.path.isabs(path) else os.path.join(base_dir, path)
        if os.path.exists(full):
            with open(full) as f:
                hits, root = json.load(f), os.path.dirname(full)
    return [dict(h, _base_dir=root) for h in hits if isinstance(h, dict)]


def _parse_entry(entry: dict, base_dir: str, dialect: str) -> JobInput:
    chains, next_id = [], 0

    def take_ids(spec: dict) -> list[str]:
        nonlocal next_id
        if "id" in spec:
            ids = _ids(spec["id"])
        else:
            ids = _letters(int(spec.get("count", 1)), next_id)
        next_id += len(ids)
        return ids

    for item in entry.get("sequences", []):
        for key, spec in item.items():
            k = key.lower()
            if k in ("protein", "proteinchain"):
                msa = spec.get("msa") if isinstance(spec.get("msa"), dict) else {}
                pre = msa.get("precomputed_msa_dir")
                unpaired = _read_text(base_dir, spec.get("unpairedMsaPath") or (os.path.join(pre, "non_pairing.a3m") if pre else None),
                                      spec.get("unpairedMsa"))  # fmt: skip
                paired = _read_text(base_dir, spec.get("pairedMsaPath") or (os.path.join(pre, "pairing.a3m") if pre else None),
                                    spec.get("pairedMsa"))  # fmt: skip
                mods = _mods(spec.get("modifications"), "ptmType", "ptmPosition")
                chains.append(ProteinChainInput(take_ids(spec), spec["sequence"].upper(), unpaired, paired, mods,
                                                _templates(spec, base_dir)))  # fmt: skip
            elif k in ("rna", "rnasequence", "dna", "dnasequence"):
                mt = const.MOL_RNA if k.startswith("rna") else const.MOL_DNA
                mods = _mods(spec.get("modifications"), "modificationType", "basePosition")
                chains.append(NucleotideChainInput(take_ids(spec), spec["sequence"].upper(), mt,
                                                   _read_text(base_dir, spec.get("unpairedMsaPath"), spec.get("unpairedMsa")), mods))  # fmt: skip
            elif k == "ligand":
                codes = spec.get("ccdCodes") or ([spec["ligand"].replace("CCD_", "")] if "ligand" in spec else [])
                chains.append(LigandChainInput(take_ids(spec), [c.upper() for c in codes], spec.get("smiles")))
            elif k == "ion":
                chains.append(LigandChainInput(take_ids(spec), [str(spec["ion"]).upper()]))
            else:
                raise ValueError(f"unknown sequence entry {key!r} in job {entry.get('name')!r}")
    bonds = []
    for pair in entry.get("bondedAtomPairs") or []:
        (c1, r1, a1), (c2, r2, a2) = pair
        bonds.append(BondedAtomPair((str(c1), int(r1), str(a1)), (str(c2), int(r2), str(a2))))
    seeds = [int(s) for s in entry.get("modelSeeds") or [0]]
    return JobInput(str(entry.get("name", "job")), chains, seeds, bonds, dialect, entry.get("userCCD"))


def parse_json_input(path_or_obj, dialect: str | None = None) -> list[JobInput]:
    """One file (or an already loaded object) -> the jobs it describes."""
    if isinstance(path_or_obj, (str, os.PathLike)):
        base_dir = os.path.dirname(os.path.abspath(path_or_obj))
        with open(path_or_obj) as f:
            obj = json.load(f)
    else:
        base_dir, obj = os.getcwd(), path_or_obj
    entries = obj if isinstance(obj, list) else [obj]
    return [_parse_entry(e, base_dir, (dialect or detect_dialect(e)).lower()) for e in entries]
