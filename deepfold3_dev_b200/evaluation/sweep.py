"""Accuracy sweeps: fold a benchmark set with one or several checkpoints, score it, follow the trajectory.

The reference tracks structure quality over a training run with a harness of shell and Python scripts around its
``inference-batch`` command (bench/README.md, bench/scripts/run_sweep.py:1-168, summarize.py, eval_trajectory.py): targets
are dealt out over the GPUs of a node, one prediction process per GPU loads the weights once and folds its share, a
re-run fills only the gaps, every seed x sample structure is scored against the experimental structure, and the tables
report the mean and the best-of-N ("oracle") per target, stratified by category and by secondary-structure class. This
module is that pipeline in one file, scored in-process with ``evaluation.compare`` (lDDT, TM-score, GDT-TS, RMSD, DockQ):

* ``discover_targets``  ``inputs/<category>/<name>.json`` + ``truth/<name>.cif`` -> ``Target`` rows with a token count
* ``plan_shards``       greedy longest-first assignment by the N^2 cost of a target, so the GPUs finish together
* ``run_sweep``         one ``inference-batch`` process per GPU (``CUDA_VISIBLE_DEVICES``, capped host threads), resumable
* ``score_step``        every ``seed-*_sample-*/model.cif`` against its truth -> ``scores.csv``
* ``summarize``         per target mean / oracle / top-ranked, per category and per fold class -> ``summary.csv``
* ``trajectory``        one row per checkpoint step and category -> ``trajectory.csv``
* ``fold_class``        alpha / beta / mixed / coil from C-alpha geometry (no DSSP binary needed)

Layout under a run directory::

    pred/step_<N>/<category>/<name>/seed-<s>_sample-<i>/model.cif   (+ ranking_scores.csv from the prediction command)
    eval/step_<N>/scores.csv, summary.csv
    trajectory.csv
"""

from __future__ import annotations

import csv
import dataclasses
import glob
import json
import os
import re
import subprocess
import sys
import time

import numpy as np

METRICS = ("lddt", "tm_score", "gdt_ts", "rmsd_trace", "dockq_mean", "ss_q3", "ss_f1_helix", "ss_f1_strand", "helix_recovery")
HIGHER_IS_BETTER = {"lddt": True, "tm_score": True, "gdt_ts": True, "rmsd_trace": False, "dockq_mean": True, "ss_q3": True,
                    "ss_f1_helix": True, "ss_f1_strand": True, "helix_recovery": True}


@dataclasses.dataclass
class Target:
    name: str
    category: str
    job: str  # path of the prediction job (JSON)
    truth: str | None  # path of the experimental structure (mmCIF), if known
    tokens: int = 0


def _count_tokens(job_path: str) -> int:
    """Residues of all polymer copies plus a flat 30 per ligand copy: only used to balance the shards."""
    try:
        with open(job_path) as f:
            obj = json.load(f)
    except (OSError, ValueError):
        return 0
    total = 0
    for entry in obj if isinstance(obj, list) else [obj]:
        for item in entry.get("sequences", []):
            for spec in item.values() if isinstance(item, dict) else []:
                if not isinstance(spec, dict):
                    continue
                copies = spec.get("count") or (len(spec["id"]) if isinstance(spec.get("id"), list) else 1)
                total += copies * (len(spec["sequence"]) if "sequence" in spec else 30)
    return total


def discover_targets(inputs_dir: str, truth_dir: str | None = None, categories=None, max_tokens: int = 0) -> list[Target]:
    out = []
    for cat in sorted(os.listdir(inputs_dir)):
        sub = os.path.join(inputs_dir, cat)
        if not os.path.isdir(sub) or (categories and cat not in categories):
            continue
        for path in sorted(glob.glob(os.path.join(sub, "*.json"))):
            name = os.path.basename(path)[:-5]
            truth = None
            if truth_dir:
                for cand in (f"{name}.cif", f"{name}.cif.gz", f"{name.lower()}.cif", f"{name.split('_')[0]}.cif"):
                    if os.path.exists(os.path.join(truth_dir, cand)):
                        truth = os.path.join(truth_dir, cand)
                        break
            t = Target(name, cat, path, truth, _count_tokens(path))
            if not max_tokens or t.tokens <= max_tokens:
                out.append(t)
    return out


def plan_shards(targets: list[Target], n: int) -> list[list[Target]]:
    """Longest first onto the least loaded shard, with cost ~ tokens^2 (the pair track dominates a prediction)."""
    shards: list[list[Target]] = [[] for _ in range(max(1, n))]
    load = [0.0] * len(shards)
    for t in sorted(targets, key=lambda t: -t.tokens):
        k = int(np.argmin(load))
        shards[k].append(t)
        load[k] += float(max(t.tokens, 1)) ** 2
    return shards


def sweep_commands(targets: list[Target], pred_root: str, params: str | None, gpus: list[int], seeds: list[int],
                   num_samples: int = 5, extra: list[str] | None = None, python: str = sys.executable):
    """``[(env, argv, inputs_file, lines)]``, one per GPU. ``inference-batch`` takes one seed per call, so the seed list
    becomes consecutive calls chained in one shell command per GPU; finished (target, seed) pairs are skipped."""
    jobs = []
    for gpu, shard in zip(gpus, plan_shards(targets, len(gpus))):
        if not shard:
            continue
        inputs = os.path.join(pred_root, f"_inputs_gpu{gpu}.txt")
        by_cat: dict[str, list[Target]] = {}
        for t in shard:
            by_cat.setdefault(t.category, []).append(t)
        calls = []
        for cat, items in sorted(by_cat.items()):
            cat_inputs = inputs.replace(".txt", f"_{cat}.txt")
            for seed in seeds:
                argv = [python, "-m", "deepfold3_dev_b200.cli", "inference-batch", "--inputs-file", cat_inputs,
                        "--output-template", os.path.join(pred_root, cat, "{name}"), "--skip-existing", "--seed", str(seed),
                        "--num-samples", str(num_samples), "--shard", "0/1"] + (["--params", params] if params else []) + list(extra or [])  # fmt: skip
                calls.append((cat_inputs, [t.job for t in items], argv))
        env = {"CUDA_VISIBLE_DEVICES": str(gpu), "OMP_NUM_THREADS": "8", "MKL_NUM_THREADS": "8", "RANK": "0", "WORLD_SIZE": "1"}
        jobs.append((env, calls))
    return jobs


def run_sweep(targets, pred_root, params, gpus, seeds, num_samples=5, extra=None, dry_run=False, log=print) -> int:
    """Launch the per-GPU processes and wait. Returns the number of failed calls. Each host process is capped at 8
    threads: without a cap every process starts one thread per core and N of them stall each other at model build."""
    os.makedirs(pred_root, exist_ok=True)
    jobs = sweep_commands(targets, pred_root, params, gpus, seeds, num_samples, extra)
    running, failed = [], 0
    for env, calls in jobs:
        for inputs, lines, _ in calls:
            with open(inputs, "w") as f:
                f.write("\n".join(lines) + "\n")
        script = " && ".join(" ".join(_quote(a) for a in argv) for _, _, argv in calls)
        log(f"gpu {env['CUDA_VISIBLE_DEVICES']}: {sum(len(c[1]) for c in calls) // max(1, len(seeds))} target(s), {len(calls)} call(s)")
        if dry_run:
            log("  " + script)
            continue
        logf = open(os.path.join(pred_root, f"_gpu{env['CUDA_VISIBLE_DEVICES']}.log"), "a")
        running.append((subprocess.Popen(["bash", "-c", script], env={**os.environ, **env}, stdout=logf, stderr=subprocess.STDOUT), logf))
    t0 = time.time()
    for proc, logf in running:
        failed += int(proc.wait() != 0)
        logf.close()
    if running:
        log(f"sweep finished in {time.time() - t0:.0f} s, {failed} failed process(es)")
    return failed


def _quote(a: str) -> str:
    return a if re.fullmatch(r"[\w@%+=:,./{}-]+", a) else "'" + a.replace("'", "'\\''") + "'"


# ------------------------------------------------------------------------------------------------------------ scoring
def fold_class(ca: np.ndarray) -> tuple[str, float, float]:
    """``(class, helix fraction, strand fraction)`` from consecutive C-alpha positions ``[L, 3]``.

    A residue counts as helical when its i..i+2, i..i+3 and i..i+4 distances are those of an alpha helix (5.5, 5.3 and
    6.4 A within 0.6), as strand when they are those of an extended chain (6.4, 9.8 and 12.4 A within 1.0 / 1.4 / 1.8);
    the classes follow the usual cut: alpha (helix >= 40 %, strand < 10 %), beta (strand >= 30 %, helix < 15 %), mixed
    (both >= 15 %), else coil. This stands in for the DSSP-based classes of the reference's tables (dssp_classify.py).
    """
    n = len(ca)
    if n < 6:
        return "coil", 0.0, 0.0
    d = lambda k: np.linalg.norm(ca[k:] - ca[:-k], axis=-1)  # noqa: E731
    d2, d3, d4 = d(2)[: n - 4], d(3)[: n - 4], d(4)[: n - 4]
    helix = (abs(d2 - 5.5) < 0.6) & (abs(d3 - 5.3) < 0.6) & (abs(d4 - 6.4) < 0.6)
    strand = (abs(d2 - 6.4) < 1.0) & (abs(d3 - 9.8) < 1.4) & (abs(d4 - 12.4) < 1.8)
    h, e = float(helix.mean()), float(strand.mean())
    if h >= 0.4 and e < 0.1:
        return "alpha", h, e
    if e >= 0.3 and h < 0.15:
        return "beta", h, e
    if h >= 0.15 and e >= 0.15:
        return "mixed", h, e
    return "coil", h, e


def _truth_class(path: str) -> str:
    from ..data.parse.mmcif import parse_mmcif

    try:
        st, _ = parse_mmcif(path, use_assembly=False)
        atoms = st.atoms
        ca = atoms[(atoms["name"] == b"CA") & atoms["is_present"]]
        return fold_class(np.stack([ca["x"], ca["y"], ca["z"]], axis=-1))[0] if len(ca) else "none"
    except Exception:  # noqa: BLE001 - a class is a label for stratification, never a reason to lose the scores
        return "unknown"


def _ranking(target_dir: str) -> dict[tuple[int, int], float]:
    path = os.path.join(target_dir, "ranking_scores.csv")
    if not os.path.exists(path):
        return {}
    with open(path) as f:
        return {(int(float(r["seed"])), int(float(r["sample"]))): float(r["ranking_score"]) for r in csv.DictReader(f)}


def score_step(pred_root: str, targets: list[Target], out_csv: str, use_assembly: bool = False, log=print) -> list[dict]:
    """Score every predicted structure of every target that has an experimental structure; writes ``out_csv``."""
    from .compare import compare_files

    rows = []
    for t in targets:
        tdir = os.path.join(pred_root, t.category, t.name)
        if not t.truth or not os.path.isdir(tdir):
            continue
        rank = _ranking(tdir)
        cls = _truth_class(t.truth)
        for sdir in sorted(glob.glob(os.path.join(tdir, "seed-*_sample-*"))):
            m = re.search(r"seed-(\d+)_sample-(\d+)$", sdir)
            cif = os.path.join(sdir, "model.cif")
            if not m or not os.path.exists(cif):
                continue
            try:
                res = compare_files(cif, t.truth, use_assembly=use_assembly)
            except Exception as exc:  # noqa: BLE001 - one unreadable file must not stop a sweep's table
                log(f"{t.name} {os.path.basename(sdir)}: not scored ({type(exc).__name__}: {exc})")
                continue
            seed, sample = int(m.group(1)), int(m.group(2))
            row = {"target": t.name, "category": t.category, "fold_class": cls, "tokens": t.tokens, "seed": seed, "sample": sample,
                   "ranking_score": rank.get((seed, sample), float("nan")), "matched_chains": res.get("matched_chains", 0)}  # fmt: skip
            row.update({k: res.get(k, float("nan")) for k in METRICS})
            rows.append(row)
    os.makedirs(os.path.dirname(os.path.abspath(out_csv)), exist_ok=True)
    with open(out_csv, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=list(rows[0]) if rows else ["target"])
        w.writeheader()
        w.writerows(rows)
    return rows


def summarize(rows: list[dict], out_csv: str | None = None) -> list[dict]:
    """Per target: mean over all structures, oracle (best of N by the metric itself) and top-ranked (the structure the
    model's own ranking score puts first; meaningless without a trained confidence head, so it is reported beside the
    confidence-free two, never instead of them). Then the mean over targets per category and per (category, fold class)."""
    per_target: dict[tuple[str, str, str], list[dict]] = {}
    for r in rows:
        per_target.setdefault((r["category"], r["fold_class"], r["target"]), []).append(r)
    table = []
    for (cat, cls, name), rs in sorted(per_target.items()):
        rec = {"category": cat, "fold_class": cls, "target": name, "n": len(rs)}
        ranked = [r for r in rs if np.isfinite(r["ranking_score"])]
        top = max(ranked, key=lambda r: r["ranking_score"]) if ranked else None
        for k in METRICS:
            vals = np.array([float(r[k]) for r in rs], dtype=float)
            vals = vals[np.isfinite(vals)]
            rec[f"{k}_mean"] = float(vals.mean()) if len(vals) else float("nan")
            rec[f"{k}_oracle"] = float((vals.max() if HIGHER_IS_BETTER[k] else vals.min())) if len(vals) else float("nan")
            rec[f"{k}_top"] = float(top[k]) if top is not None else float("nan")
        table.append(rec)
    groups: dict[tuple[str, str], list[dict]] = {}
    for rec in table:
        groups.setdefault((rec["category"], "all"), []).append(rec)
        groups.setdefault((rec["category"], rec["fold_class"]), []).append(rec)
    summary = []
    for (cat, cls), recs in sorted(groups.items()):
        row = {"category": cat, "fold_class": cls, "targets": len(recs)}
        for key in recs[0]:
            if key.endswith(("_mean", "_oracle", "_top")):
                vals = np.array([r[key] for r in recs], dtype=float)
                row[key] = float(np.nanmean(vals)) if np.isfinite(vals).any() else float("nan")
        summary.append(row)
    if out_csv:
        with open(out_csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(summary[0]) if summary else ["category"])
            w.writeheader()
            w.writerows(summary)
    return summary


def trajectory(run_dir: str, out_csv: str | None = None) -> list[dict]:
    """One row per (step, category) from the ``eval/step_*/summary.csv`` files of a run directory, ordered by step."""
    rows = []
    for path in glob.glob(os.path.join(run_dir, "eval", "step_*", "summary.csv")):
        step = int(re.search(r"step_(\d+)", path).group(1))
        with open(path) as f:
            for r in csv.DictReader(f):
                if r["fold_class"] == "all":
                    rows.append({"step": step, **{k: (v if k in ("category", "fold_class") else float(v)) for k, v in r.items()}})
    rows.sort(key=lambda r: (r["category"], r["step"]))
    if out_csv and rows:
        with open(out_csv, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=list(rows[0]))
            w.writeheader()
            w.writerows(rows)
    return rows


def resolve_checkpoint(ckpt_dir: str, step: int) -> str | None:
    """Exported weights win over the raw training checkpoint of the same step."""
    for name in (f"step_{step}.safetensors", f"checkpoint_{step}.safetensors", f"step_{step}.pt", f"checkpoint_{step}.pt"):
        if os.path.exists(os.path.join(ckpt_dir, name)):
            return os.path.join(ckpt_dir, name)
    return None
