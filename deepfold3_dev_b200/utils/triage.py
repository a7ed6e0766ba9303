"""Diagnostics for a run that misbehaves: where a non-finite value first appears, where two execution paths part,
how much per-example gradients agree, how a logged series moves, whether a prediction is a mirror image.

The reference keeps these as one-off scripts around its trainer (scripts/triage_inf.py, scripts/triage_activations.py,
scripts/measure_grad_variance.py, scripts/analyze_act_rms.py, scripts/check_chirality.py); here they are functions over
any ``nn.Module`` / run directory / pair of coordinate sets, with the ``triage`` command group on top.
"""

from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn as nn


# ---------------------------------------------------------------------------------------------------------------
# activation traces
# ---------------------------------------------------------------------------------------------------------------
@dataclass
class TraceRow:
    order: int  # position in execution order (a module called twice has two rows)
    name: str
    kind: str
    abs_max: float
    rms: float
    finite: bool


def _tensors(out):
    if isinstance(out, torch.Tensor):
        yield out
    elif isinstance(out, dict):
        for v in out.values():
            yield from _tensors(v)
    elif isinstance(out, (list, tuple)):
        for v in out:
            yield from _tensors(v)
    elif hasattr(out, "__dataclass_fields__"):
        for k in out.__dataclass_fields__:
            yield from _tensors(getattr(out, k))


def activation_trace(model: nn.Module, run, leaves_only: bool = False) -> list[TraceRow]:
    """Call ``run()`` with a forward hook on every submodule of ``model``; one row per module call in execution order
    with the largest magnitude, the RMS and whether every floating-point output was finite. Hooks are removed
    afterwards, also when ``run`` raises (the rows seen so far are attached to the exception as ``trace``)."""
    rows: list[TraceRow] = []
    handles = []

    def hook(name, kind):
        def fn(_module, _inputs, out):
            big, sq, n, ok = 0.0, 0.0, 0, True
            for t in _tensors(out):
                if not t.is_floating_point() or t.numel() == 0:
                    continue
                x = t.detach().float()
                fin = torch.isfinite(x)
                ok = ok and bool(fin.all())
                x = torch.where(fin, x, torch.zeros_like(x))
                big = max(big, float(x.abs().max()))
                sq, n = sq + float(x.pow(2).sum()), n + x.numel()
            rows.append(TraceRow(len(rows), name, kind, big, math.sqrt(sq / n) if n else 0.0, ok))

        return fn

    for name, mod in model.named_modules():
        if name and not (leaves_only and any(True for _ in mod.children())):
            handles.append(mod.register_forward_hook(hook(name, type(mod).__name__)))
    try:
        run()
    except Exception as exc:  # noqa: BLE001 - the partial trace is what the caller came for
        exc.trace = rows
        raise
    finally:
        for h in handles:
            h.remove()
    return rows


def first_nonfinite(rows: list[TraceRow]) -> TraceRow | None:
    """The first module call, in execution order, that produced a NaN or an infinity. A parent module finishes after its
    children, so the first offender is the innermost one."""
    return next((r for r in rows if not r.finite), None)


def diff_traces(a: list[TraceRow], b: list[TraceRow], rtol: float = 0.05, atol: float = 1e-6) -> list[dict]:
    """Rows of two traces of the same model (for instance kernels on and ``DF3_DISABLE_OPS`` set) whose magnitudes differ
    by more than ``rtol``; the first entry is where the two paths part. Calls are matched by (name, occurrence)."""

    def keyed(rows):
        seen: dict[str, int] = {}
        out = {}
        for r in rows:
            k = seen.get(r.name, 0)
            seen[r.name] = k + 1
            out[(r.name, k)] = r
        return out

    ka, kb = keyed(a), keyed(b)
    out = []
    for key, ra in ka.items():
        rb = kb.get(key)
        if rb is None:
            continue
        gap = abs(ra.abs_max - rb.abs_max)
        if ra.finite != rb.finite or gap > atol + rtol * max(ra.abs_max, rb.abs_max):
            out.append({"order": ra.order, "name": ra.name, "call": key[1], "abs_max_a": ra.abs_max, "abs_max_b": rb.abs_max,
                        "rms_a": ra.rms, "rms_b": rb.rms, "finite_a": ra.finite, "finite_b": rb.finite})  # fmt: skip
    return sorted(out, key=lambda d: d["order"])


def largest_activations(rows: list[TraceRow], k: int = 10) -> list[TraceRow]:
    return sorted(rows, key=lambda r: -r.abs_max)[:k]


# ---------------------------------------------------------------------------------------------------------------
# agreement of per-example gradients
# ---------------------------------------------------------------------------------------------------------------
class GradientSpread:
    """Streaming statistics of per-example gradients ``g_i``: their norms, and how well their directions agree.

    With unit vectors ``u_i = g_i / |g_i|`` the mean pairwise cosine and the resultant length follow from the running
    sum alone: ``mean_{i != j} cos = (|sum u|^2 - n) / (n^2 - n)``, ``R = |sum u| / n``. ``R`` near 1: the examples
    pull the same way and averaging them keeps the norm; ``R`` near ``1 / sqrt(n)``: directions are independent and the
    averaged gradient is mostly noise, which is when clipping each rank's gradient before the average differs most
    from clipping the average (reference: scripts/measure_grad_variance.py)."""

    def __init__(self):
        self.n, self.unit_sum, self.sum, self.norms = 0, None, None, []

    def add(self, flat_grad: torch.Tensor) -> None:
        g = flat_grad.detach().double().flatten()
        norm = float(g.norm())
        if not math.isfinite(norm) or norm == 0.0:
            return
        self.norms.append(norm)
        self.n += 1
        self.unit_sum = g / norm if self.unit_sum is None else self.unit_sum + g / norm
        self.sum = g.clone() if self.sum is None else self.sum + g

    def result(self) -> dict:
        if self.n == 0:
            return {"n": 0}
        n, s = self.n, float(self.unit_sum.norm())
        norms = np.asarray(self.norms)
        out = {"n": n, "norm_mean": float(norms.mean()), "norm_median": float(np.median(norms)), "norm_max": float(norms.max()),
               "norm_of_mean": float(self.sum.norm()) / n, "resultant_length": s / n,
               "independent_baseline": 1.0 / math.sqrt(n)}  # fmt: skip
        if n > 1:
            out["mean_pairwise_cosine"] = (s * s - n) / (n * n - n)
        return out


def flat_gradient(model: nn.Module) -> torch.Tensor:
    parts = [p.grad.flatten() for p in model.parameters() if p.grad is not None]
    return torch.cat(parts) if parts else torch.zeros(0)


# ---------------------------------------------------------------------------------------------------------------
# logged series
# ---------------------------------------------------------------------------------------------------------------
def series_summary(run_dir: str, prefix: str = "act_rms", window: int = 50, ceiling: float | None = None) -> list[dict]:
    """Every series of ``<run_dir>/logs/metrics.jsonl`` whose key starts with ``prefix``: latest value, median over the
    last ``window`` entries, and the slope of ``log(value)`` per 1000 steps over that window (fast-growing series first).
    ``ceiling`` flags series whose latest value exceeds it (the reference watches branch / stream RMS ratios against
    ``c / sqrt(depth)``, scripts/analyze_act_rms.py)."""
    path = os.path.join(run_dir, "logs", "metrics.jsonl")
    series: dict[str, list[tuple[float, float]]] = {}
    with open(path) as f:
        for line in f:
            try:
                row = json.loads(line)
            except ValueError:
                continue
            step = row.get("step", row.get("train/step"))
            if step is None:
                continue
            for k, v in row.items():
                name = k.split("/", 1)[1] if k.startswith(("train/", "eval/")) and k.split("/", 1)[1].startswith(prefix) else k
                if name.startswith(prefix) and isinstance(v, (int, float)) and math.isfinite(v):
                    series.setdefault(name, []).append((float(step), float(v)))
    out = []
    for name, pts in series.items():
        pts = sorted(pts)[-window:]
        steps, vals = np.asarray([p[0] for p in pts]), np.asarray([p[1] for p in pts])
        slope = 0.0
        if len(pts) >= 3 and np.ptp(steps) > 0 and (vals > 0).all():
            slope = float(np.polyfit(steps, np.log(vals), 1)[0] * 1000.0)
        row = {"series": name, "latest": float(vals[-1]), "median": float(np.median(vals)), "log_slope_per_1k_steps": slope,
               "points": len(pts)}  # fmt: skip
        if ceiling is not None:
            row["above_ceiling"] = bool(vals[-1] > ceiling)
        out.append(row)
    return sorted(out, key=lambda r: -r["log_slope_per_1k_steps"])


# ---------------------------------------------------------------------------------------------------------------
# the distogram head against the true distances
# ---------------------------------------------------------------------------------------------------------------
@torch.no_grad()
def distogram_agreement(model, feats: dict, num_recycles: int = 1, seed: int = 0, near: float = 20.0) -> dict:
    """Trunk and distogram head only (no diffusion) on one example with ground truth: how often the most likely bin is
    the true one (or next to it), the cross-entropy, and the mean absolute error of the expected distance over pairs
    closer than ``near`` angstroms. A trunk that has learnt the fold shows here long before samples look right
    (reference: scripts/check_distogram.py, there as heat maps). Returns the ``[N, N]`` true and expected distance
    maps too, for plotting."""
    was_training = model.training
    model.eval()
    try:
        trunk = model.run_evoformer(feats, num_recycles, seed=seed)
        pair = trunk[0]["pair"]
        head = model.distogram_head
        logits = head(pair).float()
        expected = head.expected_distance(pair).float()
    finally:
        model.train(was_training)
    while logits.dim() > 3:  # drop a leading batch axis of one
        logits, expected = logits[0], expected[0]
    n = logits.shape[0]
    ar = torch.arange(n, device=logits.device)
    rep = feats["token_to_rep_atom"].reshape(-1)[:n].long()
    pos = feats["atom_gt_positions"].reshape(-1, *feats["atom_gt_positions"].shape[-2:])[:n][ar, rep].float()
    ok = feats["atom_gt_mask"].reshape(-1, feats["atom_gt_mask"].shape[-1])[:n][ar, rep].bool()
    d = torch.cdist(pos, pos)
    valid = ok[:, None] & ok[None] & ~torch.eye(n, dtype=torch.bool, device=d.device)
    breaks = torch.linspace(head.first_break, head.last_break, head.num_bins - 1, device=d.device)
    target = torch.bucketize(d, breaks)
    pred = logits.argmax(-1)
    count = int(valid.sum())
    if count == 0:
        return {"pairs": 0}
    nll = torch.nn.functional.cross_entropy(logits[valid], target[valid])
    close = valid & (d < near)
    return {"pairs": count, "bin_accuracy": float((pred == target)[valid].float().mean()),
            "bin_within_one": float(((pred - target).abs() <= 1)[valid].float().mean()), "cross_entropy": float(nll),
            "uniform_cross_entropy": math.log(head.num_bins),
            "mae_expected_distance_near": float((expected - d).abs()[close].mean()) if bool(close.any()) else float("nan"),
            "true_distance": d.cpu(), "expected_distance": expected.cpu()}  # fmt: skip


# ---------------------------------------------------------------------------------------------------------------
# handedness of a prediction
# ---------------------------------------------------------------------------------------------------------------
def _pseudo_dihedrals(ca: np.ndarray) -> np.ndarray:
    b0, b1, b2 = ca[1:-2] - ca[:-3], ca[2:-1] - ca[1:-2], ca[3:] - ca[2:-1]
    n1, n2 = np.cross(b0, b1), np.cross(b1, b2)
    m = np.cross(n1, b1 / np.linalg.norm(b1, axis=-1, keepdims=True).clip(1e-9))
    return np.arctan2((m * n2).sum(-1), (n1 * n2).sum(-1))


def handedness(pred_ca: np.ndarray, ref_ca: np.ndarray) -> dict:
    """Is ``pred_ca`` ``[L, 3]`` the mirror image of ``ref_ca`` (same residues, same order)?

    ``improper_fit``: the best orthogonal map between the two point sets has determinant -1, i.e. a reflection fits
    better than a rotation. ``dihedral_sign_match``: fraction of 4-residue windows whose C-alpha pseudo-dihedral has the
    sign it has in the reference (right-handed helices sit near +50 degrees, their mirror image near -50); windows with a
    nearly flat reference dihedral are left out. ``rmsd_proper`` / ``rmsd_mirrored``: RMSD after the best rotation of
    the prediction and of its mirror image (reference: scripts/check_chirality.py, metrics (a) and (b))."""
    from ..evaluation.metrics import rmsd

    p, r = np.asarray(pred_ca, np.float64), np.asarray(ref_ca, np.float64)
    if p.shape != r.shape or p.ndim != 2 or p.shape[0] < 4:
        raise ValueError("handedness needs two [L, 3] traces of the same residues, L >= 4")
    h = (p - p.mean(0)).T @ (r - r.mean(0))
    u, _, vt = np.linalg.svd(h)
    improper = bool(np.linalg.det(vt.T @ u.T) < 0)
    dp, dr = _pseudo_dihedrals(p), _pseudo_dihedrals(r)
    keep = np.abs(dr) > math.radians(10) if len(dr) else np.zeros(0, bool)
    match = float((np.sign(dp[keep]) == np.sign(dr[keep])).mean()) if keep.any() else float("nan")
    mirrored = p * np.array([-1.0, 1.0, 1.0])
    return {"improper_fit": improper, "dihedral_sign_match": match, "windows": int(keep.sum()),
            "rmsd_proper": float(rmsd(p, r)), "rmsd_mirrored": float(rmsd(mirrored, r)),
            "mirror_image": bool(improper and (math.isnan(match) or match < 0.5))}  # fmt: skip


def handedness_of_files(pred_path: str, ref_path: str) -> list[dict]:
    """``handedness`` per matched polymer chain of two structure files (chains matched as in ``evaluate``)."""
    from ..data.parse.mmcif import parse_mmcif
    from ..evaluation.compare import match_chains, matched_atoms

    pred, _ = parse_mmcif(pred_path, use_assembly=False)
    true, _ = parse_mmcif(ref_path, use_assembly=False)
    out = []
    for k, pair in enumerate(match_chains(pred, true)):
        P, T, _, _, trace = matched_atoms(pred, true, [pair])
        if int(trace.sum()) >= 4:
            out.append({"chain_pair": k, "asym_pred": pair[0]["asym"], "asym_ref": pair[1]["asym"],
                        "residues": int(trace.sum()), **handedness(P[trace], T[trace])})  # fmt: skip
    return out
