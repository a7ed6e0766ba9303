"""Job descriptions in four JSON dialects -> ``JobInput`` (reference: data/parse/json_input.py:56-1415).

* ``alphafold3``: ``{"name", "modelSeeds", "sequences": [{"protein"|"rna"|"dna"|"ligand": {"id", ...}}]}`` with MSAs as
  inline A3M text or paths, inline ``templates`` or a ``templatesPath``, ``bondedAtomPairs``, ``userCCD`` / ``userCCDPath``
* ``alphafoldserver``: jobs with ``proteinChain`` / ``rnaSequence`` / ``dnaSequence`` / ``ligand`` / ``ion`` entries carrying
  ``count``; no alignments in the file (they are searched when the caller passes ``msa_search``), a random seed when
  ``modelSeeds`` is empty
* ``protenix``: ``proteinChain`` / ``dnaSequence`` | ``dnaChain`` / ``rnaSequence`` | ``rnaChain`` with ``count``,
  ``msa.precomputed_msa_dir`` (``pairing.a3m``, ``non_pairing.a3m``), ``pairedMsaPath`` / ``unpairedMsaPath``,
  ``templatesPath`` (JSON hit list or HHsearch ``.hhr``), ``ligand`` as ``CCD_<code>`` or a SMILES string
* ``deepfold3``: the union of the key styles above

The dialect is taken from a ``"dialect"`` field or detected from the keys. Paths are relative to the JSON file.
Malformed optional parts (a modification without a position, a bond that is not two ``[chain, residue, atom]``
triples, an unreadable alignment file, a bad ``maxTemplateDate``) are skipped with a warning, as the reference does; a
job without any chain, an unknown sequence key or an unknown ``msa_pairing`` mode is an error. ``maxTemplateDate`` drops
template hits whose ``releaseDate`` is later (hits without a date are kept: they cannot be checked).

MSA search is a process boundary and off by default: a protein chain without an alignment gets a single-row alignment
(its own sequence). ``parse_json_input(..., msa_search=fn)`` calls ``fn(sequences) -> [{"unpaired": a3m, "paired": a3m
or None, "templates": [hit dicts]}]`` once per job for the distinct protein sequences that have none
(``msa_search_from_server`` / ``msa_search_local`` build such functions).
"""

from __future__ import annotations

import dataclasses
import datetime
import json
import logging
import os
import random

from .. import const

logger = logging.getLogger(__name__)

DIALECTS = ("alphafold3", "alphafoldserver", "protenix", "deepfold3")
MSA_PAIRING_MODES = ("auto", "precomputed", "species", "none")
_PROTEIN_KEYS = ("protein", "proteinchain")
_RNA_KEYS = ("rna", "rnasequence", "rnachain")
_DNA_KEYS = ("dna", "dnasequence", "dnachain")


@dataclasses.dataclass
class ProteinChainInput:
    ids: list[str]
    sequence: str
    unpaired_msa: str | None = None  # A3M text
    paired_msa: str | None = None
    modifications: list[tuple[str, int]] = dataclasses.field(default_factory=list)  # (CCD code, 1-based position)
    templates: list[dict] = dataclasses.field(default_factory=list)
    mol_type: int = const.MOL_PROTEIN
    description: str | None = None


@dataclasses.dataclass
class NucleotideChainInput:
    ids: list[str]
    sequence: str
    mol_type: int = const.MOL_RNA
    unpaired_msa: str | None = None
    modifications: list[tuple[str, int]] = dataclasses.field(default_factory=list)
    description: str | None = None


@dataclasses.dataclass
class LigandChainInput:
    ids: list[str]
    ccd_codes: list[str] = dataclasses.field(default_factory=list)
    smiles: str | None = None
    mol_type: int = const.MOL_NONPOLYMER
    description: str | None = None


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
    max_template_date: str | None = None  # YYYY-MM-DD
    description: str | None = None

    @property
    def num_chains(self) -> int:
        return sum(len(c.ids) for c in self.chains)


def _ids(raw) -> list[str]:
    return [raw] if isinstance(raw, str) else list(raw)


def _letters(n: int, start: int) -> list[str]:
    from ...io.mmcif import asym_id_to_chain_name

    return [asym_id_to_chain_name(start + i) for i in range(n)]


def _resolve(base_dir: str, path: str | None) -> str | None:
    if not path:
        return None
    return path if os.path.isabs(path) else os.path.join(base_dir, path)


def _read_text(base_dir: str, path: str | None, inline: str | None) -> str | None:
    """Text behind a path (preferred when given) or an inline string; ``None`` when absent, empty or unreadable."""
    if path:
        full = _resolve(base_dir, path)
        try:
            with open(full) as f:
                return f.read()
        except OSError as exc:
            logger.warning("cannot read %s: %s", full, exc)
            return None
    if inline and inline.strip():
        return inline
    return None


def _mods(raw) -> list[tuple[str, int]]:
    """``[(component code, 1-based position)]`` from the AF3 (``ptmType`` / ``ptmPosition``), nucleotide
    (``modificationType`` / ``basePosition``) and Protenix (``modificationPosition``) spellings; bad entries are skipped."""
    out = []
    for m in raw or []:
        if not isinstance(m, dict):
            logger.warning("modification skipped (not an object): %r", m)
            continue
        code = m.get("ptmType") or m.get("modificationType")
        pos = next((m[k] for k in ("ptmPosition", "basePosition", "modificationPosition") if m.get(k) is not None), None)
        try:
            if not code:
                raise ValueError("no type")
            out.append((str(code).strip().upper().removeprefix("CCD_"), int(pos)))
        except (TypeError, ValueError):
            logger.warning("modification skipped (needs a type and an integer position): %r", m)
    return out


def _bonds(raw) -> list[BondedAtomPair]:
    out = []
    for pair in raw or []:
        try:
            (c1, r1, a1), (c2, r2, a2) = pair
            out.append(BondedAtomPair((str(c1), int(r1), str(a1)), (str(c2), int(r2), str(a2))))
        except (TypeError, ValueError):
            logger.warning("bondedAtomPairs entry skipped (want [[chain, residue, atom], [chain, residue, atom]]): %r", pair)
    return out


def _date(raw) -> str | None:
    if raw in (None, ""):
        return None
    try:
        return datetime.date.fromisoformat(str(raw).strip()).isoformat()
    except ValueError:
        logger.warning("maxTemplateDate %r ignored (want YYYY-MM-DD)", raw)
        return None


def _user_ccd(base_dir: str, inline: str | None, path: str | None) -> str | None:
    if inline and path:
        logger.warning("userCCD and userCCDPath both given: the inline text is used")
    if inline:
        return inline
    if path:
        full = _resolve(base_dir, path)
        try:
            if full.endswith(".gz"):
                import gzip

                with gzip.open(full, "rt") as f:
                    return f.read()
            with open(full) as f:
                return f.read()
        except OSError as exc:
            logger.warning("userCCDPath %s not read: %s", full, exc)
    return None


def detect_dialect(entry: dict) -> str:
    if isinstance(entry.get("dialect"), str) and entry["dialect"].lower() in DIALECTS:
        return entry["dialect"].lower()
    keys = set()
    for s in entry.get("sequences", []):
        keys.update(k.lower() for k in s)
    if keys & {"protein", "rna", "dna"}:
        return "alphafold3"
    if "ligand" in keys and any(isinstance(s.get("ligand"), dict) and ("ccdCodes" in s["ligand"] or "id" in s["ligand"])
                                for s in entry.get("sequences", [])):  # fmt: skip
        return "alphafold3"
    if keys & {"proteinchain", "rnasequence", "dnasequence", "rnachain", "dnachain", "ion"}:
        fields = ("msa", "pairedMsaPath", "unpairedMsaPath", "templatesPath")
        has_msa = any(f in v for s in entry.get("sequences", []) for v in s.values() if isinstance(v, dict) for f in fields)
        return "protenix" if has_msa else "alphafoldserver"
    return "deepfold3"


def _templates(spec: dict, base_dir: str) -> list[dict]:
    """Inline ``templates``, or the hits behind ``templatesPath``: a JSON hit list, or an HHsearch ``.hhr`` file whose
    hits become ``{"pdbId", "chainId", "queryIndices", "templateIndices"}`` (the structure file is looked up later in
    the local mmCIF mirror). Every hit remembers the directory relative paths start from."""
    hits, root = list(spec.get("templates") or []), base_dir
    path = _resolve(base_dir, spec.get("templatesPath"))
    if not hits and path:
        if not os.path.exists(path):
            logger.warning("templatesPath %s not found", path)
        elif path.endswith(".hhr"):
            from .hhr import parse_hhr

            with open(path) as f:
                for h in parse_hhr(f.read()):
                    pairs = [(q, t) for q, t in zip(h.indices_query, h.indices_hit) if q != -1 and t != -1]
                    hits.append({"pdbId": h.pdb_id, "chainId": h.chain_id, "queryIndices": [q for q, _ in pairs],
                                 "templateIndices": [t for _, t in pairs], "eValue": h.e_value,
                                 "templateSequence": h.hit_sequence.replace("-", "")})  # fmt: skip
            root = os.path.dirname(path)
        else:
            with open(path) as f:
                hits, root = json.load(f), os.path.dirname(path)
    return [dict(h, _base_dir=root) for h in hits if isinstance(h, dict)]


def _filter_templates_by_date(job: JobInput) -> None:
    if not job.max_template_date:
        return
    for c in job.chains:
        hits = getattr(c, "templates", None)
        if hits:
            keep = [h for h in hits if not h.get("releaseDate") or str(h["releaseDate"])[:10] <= job.max_template_date]
            if len(keep) != len(hits):
                logger.info("%d template hit(s) released after %s dropped", len(hits) - len(keep), job.max_template_date)
            c.templates = keep


def _parse_entry(entry: dict, base_dir: str, dialect: str) -> JobInput:
    chains, next_id = [], 0
    name = str(entry.get("name", "job"))

    def take_ids(spec: dict) -> list[str]:
        nonlocal next_id
        if "id" in spec:
            ids = _ids(spec["id"])
        else:
            ids = _letters(int(spec.get("count", 1)), next_id)
        next_id += len(ids)
        return ids

    def msa_paths(spec: dict):
        """(unpaired path, paired path) with Protenix's ``msa.precomputed_msa_dir`` as the fallback."""
        unpaired, paired = spec.get("unpairedMsaPath"), spec.get("pairedMsaPath")
        pre = spec["msa"].get("precomputed_msa_dir") if isinstance(spec.get("msa"), dict) else None
        if pre and not unpaired and not paired:
            full = _resolve(base_dir, pre)
            if os.path.isfile(os.path.join(full, "non_pairing.a3m")):
                unpaired = os.path.join(full, "non_pairing.a3m")
            if os.path.isfile(os.path.join(full, "pairing.a3m")):
                paired = os.path.join(full, "pairing.a3m")
        return unpaired, paired

    for item in entry.get("sequences", []):
        for key, spec in item.items():
            k = key.lower()
            if k in _PROTEIN_KEYS:
                unpaired, paired = msa_paths(spec)
                chains.append(ProteinChainInput(take_ids(spec), spec["sequence"].upper(), _read_text(base_dir, unpaired, spec.get("unpairedMsa")),
                                                _read_text(base_dir, paired, spec.get("pairedMsa")), _mods(spec.get("modifications")),
                                                _templates(spec, base_dir), description=spec.get("description")))  # fmt: skip
            elif k in _RNA_KEYS or k in _DNA_KEYS:
                unpaired, _ = msa_paths(spec)
                chains.append(NucleotideChainInput(take_ids(spec), spec["sequence"].upper(), const.MOL_RNA if k in _RNA_KEYS else const.MOL_DNA,
                                                   _read_text(base_dir, unpaired, spec.get("unpairedMsa")), _mods(spec.get("modifications")),
                                                   description=spec.get("description")))  # fmt: skip
            elif k == "ligand":
                codes, smiles = spec.get("ccdCodes"), spec.get("smiles")
                raw = spec.get("ligand")
                if not codes and isinstance(raw, str) and raw:
                    if raw.startswith("CCD_"):
                        codes = [raw[4:]]
                    elif dialect == "alphafoldserver":
                        codes = [raw]  # the server format names components without the prefix, too
                    else:
                        smiles = smiles or raw  # Protenix: anything else is a SMILES string
                if not codes and not smiles:
                    logger.warning("ligand entry without ccdCodes, ligand or smiles skipped in job %r", name)
                    continue
                chains.append(LigandChainInput(take_ids(spec), [str(c).upper() for c in codes or []], smiles,
                                               description=spec.get("description")))  # fmt: skip
            elif k == "ion":
                chains.append(LigandChainInput(take_ids(spec), [str(spec["ion"]).upper().removeprefix("CCD_")]))
            else:
                raise ValueError(f"unknown sequence entry {key!r} in job {name!r}")
    if not chains:
        raise ValueError(f"no chains found in job {name!r}")
    raw_seeds = entry.get("modelSeeds") or []
    if raw_seeds:
        seeds = [int(x) for x in raw_seeds]
    else:  # the server format draws a seed; the file formats fall back to a fixed one
        seeds = [random.randint(0, 2**32 - 1)] if dialect == "alphafoldserver" else [42]
    job = JobInput(name, chains, seeds, _bonds(entry.get("bondedAtomPairs")), dialect,
                   _user_ccd(base_dir, entry.get("userCCD"), entry.get("userCCDPath")), _date(entry.get("maxTemplateDate")),
                   entry.get("description"))  # fmt: skip
    _filter_templates_by_date(job)
    return job


def _fill_missing_alignments(job: JobInput, msa_search) -> None:
    todo = list(dict.fromkeys(c.sequence for c in job.chains if isinstance(c, ProteinChainInput) and not c.unpaired_msa and not c.paired_msa))
    if not todo:
        return
    found = dict(zip(todo, msa_search(todo)))
    for c in job.chains:
        if isinstance(c, ProteinChainInput) and not c.unpaired_msa and not c.paired_msa and c.sequence in found:
            res = found[c.sequence]
            c.unpaired_msa, c.paired_msa = res.get("unpaired"), res.get("paired")
            if not c.templates and res.get("templates"):
                c.templates = list(res["templates"])
    _filter_templates_by_date(job)


def parse_json_input(path_or_obj, dialect: str | None = None, msa_search=None, msa_pairing: str = "auto") -> list[JobInput]:
    """One file (or an already loaded object) -> the jobs it describes."""
    if msa_pairing not in MSA_PAIRING_MODES:
        raise ValueError(f"msa_pairing must be one of {MSA_PAIRING_MODES}, got {msa_pairing!r}")
    if isinstance(path_or_obj, (str, os.PathLike)):
        base_dir = os.path.dirname(os.path.abspath(path_or_obj))
        with open(path_or_obj) as f:
            obj = json.load(f)
    else:
        base_dir, obj = os.getcwd(), path_or_obj
    entries = obj if isinstance(obj, list) else [obj]
    jobs = [_parse_entry(e, base_dir, (dialect or detect_dialect(e)).lower()) for e in entries]
    if msa_search is not None:
        for job in jobs:
            _fill_missing_alignments(job, msa_search)
    return jobs


def msa_search_from_server(cache_dir: str | None = None, host: str | None = None):
    """A ``msa_search`` function over the ColabFold MMseqs2 API: unpaired alignments per sequence, and paired ones when
    a job has more than one distinct protein sequence."""
    from ..msa import search

    cache = search.MsaCache(os.path.expanduser(cache_dir)) if cache_dir else None
    kw = {"host": host} if host else {}

    def run(sequences: list[str]) -> list[dict]:
        unpaired = search.search_server(sequences, cache, **kw)
        paired = search.search_server(sequences, cache, pairing=True, **kw) if len(sequences) > 1 else [None] * len(sequences)
        return [{"unpaired": u, "paired": p} for u, p in zip(unpaired, paired)]

    return run


def msa_search_local(settings, cache_dir: str | None = None, paired: bool = True):
    """A ``msa_search`` function over the staged local MMseqs2 pipeline (``data/msa/mmseqs_pipeline.py``); template hits
    come back as ``{"pdbId", "chainId", "queryIndices", "templateIndices"}`` from the m8 table's CIGAR strings."""
    from ..msa import mmseqs_pipeline as mp
    from ..msa import search
    from ..templates import cigar_to_index_pairs

    cache = search.MsaCache(os.path.expanduser(cache_dir)) if cache_dir else None

    def run(sequences: list[str]) -> list[dict]:
        mono = mp.search_monomer_batch(sequences, settings, cache)
        blocks = mp.search_pair_batch([sequences], settings, cache)[0] if paired and len(sequences) > 1 else [None] * len(sequences)
        out = []
        for res, pair in zip(mono, blocks):
            hits = []
            for per_query in mp.parse_m8(res["m8"]).values():
                for h in per_query:
                    pdb, _, chain = h.target.partition("_")
                    q, t = cigar_to_index_pairs(h.cigar, h.q_start, h.t_start)  # 1-based starts, as in the m8 table
                    hits.append({"pdbId": pdb.upper(), "chainId": chain or "A", "queryIndices": q, "templateIndices": t, "eValue": h.evalue})
            out.append({"unpaired": res["a3m"], "paired": pair, "templates": hits})
        return out

    return run
