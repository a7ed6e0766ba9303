"""Directory of mmCIF files -> ``structures/<id>.npz`` + ``manifest.json`` + ``sequences.fasta``.

Reference: scripts/prepare.py:316-1546 (sub-commands) over data/prepare/{structure,filters,manifest,sequences}.py.
One entry is parsed, checked against the entry-level rules, its chains are marked by the chain-level rules, and the
structure and record are written; the manifest and the FASTA of unique polymer sequences (keyed by ``msa_id``, the
input of the MSA search step) are written once at the end. Entries are independent, so the work fans out over processes.
"""

from __future__ import annotations

import json
import os
from concurrent.futures import ProcessPoolExecutor

from .. import const
from ..parse.mmcif import parse_mmcif
from ..types import Record, Structure, save_manifest
from .filters import StructureFilterConfig, filter_structure, filter_structure_metadata

_CIF_SUFFIXES = (".cif", ".cif.gz", ".cif.zst", ".mmcif")


def find_mmcif_files(root: str) -> list[str]:
    out = []
    for base, _dirs, files in os.walk(root):
        out.extend(os.path.join(base, f) for f in files if f.lower().endswith(_CIF_SUFFIXES))
    return sorted(out)


def chain_sequences(st: Structure, rec: Record) -> dict[str, str]:
    """``msa_id`` -> one-letter sequence for the polymer chains (canonical when the entry gave one)."""
    letters = {v: k for k, v in const.PROTEIN_1TO3.items()}
    letters.update({"A": "A", "G": "G", "C": "C", "U": "U", "DA": "A", "DG": "G", "DC": "C", "DT": "T", "N": "N"})
    out = {}
    for ci in rec.chains:
        if ci.mol_type == const.MOL_NONPOLYMER:
            continue
        seq = (st.chain_canonical_seqs or {}).get(ci.chain_id)
        if seq is None:
            c = st.chains[ci.chain_id]
            res = st.residues[int(c["res_idx"]) : int(c["res_idx"]) + int(c["res_num"])]
            seq = "".join(letters.get(const.RES_TYPE_INDEX_TO_NAME[int(t)], "X") for t in res["res_type"])
        out[str(ci.msa_id)] = seq
    return out


def process_entry(path: str, out_dir: str, cfg: StructureFilterConfig | None = None, use_assembly: bool = True) -> dict:
    """Returns ``{"id", "status": "ok"|"rejected"|"error", "reason", "record", "sequences"}`` (JSON-friendly)."""
    cfg = cfg or StructureFilterConfig()
    try:
        st, rec = parse_mmcif(path, use_assembly=use_assembly, max_chains=cfg.max_chains,
                              drop_crystallization_aids=cfg.drop_crystallization_aids)
    except Exception as exc:  # noqa: BLE001 - one unreadable entry must not stop the run
        return {"id": os.path.basename(path), "status": "error", "reason": f"{type(exc).__name__}: {exc}"}
    polymers = sum(1 for c in rec.chains if c.mol_type != const.MOL_NONPOLYMER)
    why = filter_structure_metadata(rec.structure_info, cfg, len(rec.chains), len(st.residues), polymers)
    if why is not None:
        return {"id": rec.id, "status": "rejected", "reason": why}
    rec, reasons = filter_structure(st, rec, cfg)
    if not any(c.valid for c in rec.chains):
        return {"id": rec.id, "status": "rejected", "reason": "no valid chain: " + "; ".join(f"{k}: {v}" for k, v in reasons.items())}
    os.makedirs(os.path.join(out_dir, "structures"), exist_ok=True)
    st.save(os.path.join(out_dir, "structures", f"{rec.id}.npz"))
    return {"id": rec.id, "status": "ok", "reason": reasons, "record": rec.to_dict(), "sequences": chain_sequences(st, rec)}


def _job(args):
    return process_entry(*args)


def prepare_directory(src: str, out_dir: str, cfg: StructureFilterConfig | None = None, workers: int = 1,
                      use_assembly: bool = True, limit: int = 0) -> dict:  # fmt: skip
    """Run every entry under ``src``; writes the manifest, the FASTA and ``prepare_report.json``. Returns the counts."""
    files = find_mmcif_files(src)
    if limit:
        files = files[:limit]
    os.makedirs(out_dir, exist_ok=True)
    jobs = [(f, out_dir, cfg, use_assembly) for f in files]
    if workers > 1:
        with ProcessPoolExecutor(workers) as pool:
            results = list(pool.map(_job, jobs, chunksize=4))
    else:
        results = [_job(j) for j in jobs]
    records, seqs, report = [], {}, {"ok": 0, "rejected": 0, "error": 0, "details": {}}
    for r in results:
        report[r["status"]] += 1
        if r["status"] == "ok":
            records.append(Record.from_dict(r["record"]))
            seqs.update(r["sequences"])
        if r.get("reason"):
            report["details"][r["id"]] = r["reason"]
    save_manifest(records, os.path.join(out_dir, "manifest.json"))
    with open(os.path.join(out_dir, "sequences.fasta"), "w") as f:
        for key in sorted(seqs):
            f.write(f">{key}\n{seqs[key]}\n")
    with open(os.path.join(out_dir, "prepare_report.json"), "w") as f:
        json.dump(report, f, indent=1)
    return {k: report[k] for k in ("ok", "rejected", "error")}


def load_fasta(path: str) -> dict[str, str]:
    out, key = {}, None
    with open(path) as f:
        for line in f:
            line = line.strip()
            if line.startswith(">"):
                key = line[1:].split()[0]
                out[key] = ""
            elif key is not None:
                out[key] += line
    return out
