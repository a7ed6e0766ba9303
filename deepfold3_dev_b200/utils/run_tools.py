"""Run triage helpers: what is inside a checkpoint, and how a run is doing
(reference: repo-root scripts analyze_checkpoint.py, run_status.py, triage_inf.py).

``checkpoint_report`` groups parameters by top-level module and reports sizes, norms, non-finite counts and, when the
checkpoint carries an EMA shadow, how far the shadow is from the live weights. ``run_status`` reads ``logs/metrics.jsonl``
of a run directory and summarises progress, throughput, the loss trend and skipped steps.
"""

from __future__ import annotations

import json
import os

import torch

from ..compat import torch_load_compat


def checkpoint_report(path: str, depth: int = 2) -> dict:
    blob = torch_load_compat(path) if path.endswith(".pt") else None
    if blob is None:
        from safetensors.torch import load_file

        blob = {"model": load_file(path)}
    model = blob["model"] if isinstance(blob, dict) and "model" in blob else blob
    ema = (blob.get("ema") or {}) if isinstance(blob, dict) else {}
    ema = ema.get("shadow", ema) if isinstance(ema, dict) else {}
    groups: dict[str, dict] = {}
    bad = []
    for name, t in model.items():
        if not torch.is_tensor(t):
            continue
        key = ".".join(name.split(".")[:depth])
        g = groups.setdefault(key, {"tensors": 0, "parameters": 0, "sq": 0.0, "max_abs": 0.0, "ema_sq_diff": 0.0, "has_ema": False})
        f = t.float()
        n_bad = int((~torch.isfinite(f)).sum())
        if n_bad:
            bad.append({"name": name, "non_finite": n_bad})
        g["tensors"] += 1
        g["parameters"] += t.numel()
        g["sq"] += float(torch.nan_to_num(f).pow(2).sum())
        g["max_abs"] = max(g["max_abs"], float(torch.nan_to_num(f).abs().max()) if t.numel() else 0.0)
        if isinstance(ema, dict) and name in ema and torch.is_tensor(ema[name]) and ema[name].shape == t.shape:
            g["ema_sq_diff"] += float((ema[name].float() - f).pow(2).sum())
            g["has_ema"] = True
    rows = []
    for key, g in sorted(groups.items()):
        row = {"module": key, "tensors": g["tensors"], "parameters": g["parameters"], "norm": g["sq"] ** 0.5, "max_abs": g["max_abs"]}
        if g["has_ema"]:
            row["ema_distance"] = g["ema_sq_diff"] ** 0.5
        rows.append(row)
    meta = {k: blob.get(k) for k in ("global_step", "effective_step", "epoch", "best_eval_loss", "snapshot_kind")} if isinstance(blob, dict) else {}
    return {"path": path, "meta": {k: v for k, v in meta.items() if v is not None},
            "total_parameters": sum(g["parameters"] for g in groups.values()), "non_finite": bad, "modules": rows}  # fmt: skip


def run_status(run_dir: str, window: int = 100) -> dict:
    path = os.path.join(run_dir, "logs", "metrics.jsonl")
    if not os.path.exists(path):
        path = os.path.join(run_dir, "metrics.jsonl")
    rows = []
    with open(path) as f:
        for line in f:
            try:
                rows.append(json.loads(line))
            except json.JSONDecodeError:
                continue  # a line cut off by a crash
    if not rows:
        return {"run": run_dir, "rows": 0}
    loss_key = next((k for k in ("train/loss", "loss", "train/total_loss", "total_loss") if any(k in r for r in rows)), None)
    out = {"run": run_dir, "rows": len(rows), "first_step": rows[0].get("step"), "last_step": rows[-1].get("step")}
    timed = [r for r in rows if "time" in r and "step" in r]
    if len(timed) >= 2 and timed[-1]["time"] > timed[0]["time"]:
        recent = timed[-window:]
        span = recent[-1]["time"] - recent[0]["time"]
        if span > 0:
            out["steps_per_hour"] = 3600.0 * (recent[-1]["step"] - recent[0]["step"]) / span
    if loss_key:
        losses = [float(r[loss_key]) for r in rows if isinstance(r.get(loss_key), (int, float))]
        if losses:
            k = max(1, min(window, len(losses) // 2))
            out["loss_key"], out["loss_last"] = loss_key, losses[-1]
            out["loss_recent_mean"], out["loss_earlier_mean"] = sum(losses[-k:]) / k, sum(losses[:k]) / k
            out["non_finite_losses"] = sum(1 for x in losses if x != x or x in (float("inf"), float("-inf")))
    skipped = [r.get("skipped_steps") or r.get("train/skipped_steps") for r in rows if ("skipped_steps" in r or "train/skipped_steps" in r)]
    if skipped:
        out["skipped_steps"] = skipped[-1]
    ckpts = sorted(f for f in os.listdir(run_dir) if f.endswith(".pt")) if os.path.isdir(run_dir) else []
    out["checkpoints"] = ckpts[-3:]
    return out
