#!/usr/bin/env python
"""Bar charts of the benchmark JSON files this directory writes.

    python benchmarks/plot_results.py bench_results/modules_forward.json [more.json ...] [--out plots/]

Recognised inputs: the row lists of ``bench_modules.py`` (kernels against PyTorch per module, with the speed-up printed
on the bars), ``bench_pairformer_stack.py`` (both arms per token count when rows of both are given) and ``verify.py``
(errors of the two bf16 paths against the fp32 oracle, log scale). One PNG per input file, named after it. Counterpart
of the reference's benchmarks/plot_results.py.
"""

from __future__ import annotations

import argparse
import json
import os


def _bars(ax, labels, series: dict, ylabel: str, log: bool = False, annotate=None):
    import numpy as np

    x = np.arange(len(labels))
    width = 0.8 / max(1, len(series))
    for k, (name, values) in enumerate(series.items()):
        bars = ax.bar(x + (k - (len(series) - 1) / 2) * width, values, width, label=name)
        if annotate is not None and k == 0:
            for rect, text in zip(bars, annotate):
                ax.annotate(text, (rect.get_x() + rect.get_width() / 2, rect.get_height()), ha="center", va="bottom", fontsize=7)
    ax.set_xticks(x)
    ax.set_xticklabels(labels, rotation=40, ha="right", fontsize=8)
    ax.set_ylabel(ylabel)
    if log:
        ax.set_yscale("log")
    ax.legend(fontsize=8)


def plot_file(path: str, out_dir: str) -> str:
    try:
        import matplotlib

        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError as exc:
        raise RuntimeError("plotting needs matplotlib") from exc

    with open(path) as f:
        rows = json.load(f)
    if not rows:
        raise ValueError(f"{path}: no rows")
    fig, ax = plt.subplots(figsize=(max(6, 0.7 * len(rows) + 2), 4))
    first = rows[0]
    if "ours_ms" in first:  # bench_modules
        labels = [r["module"] for r in rows]
        _bars(ax, labels, {"kernels": [r["ours_ms"] or 0 for r in rows], "PyTorch": [r["eager_ms"] or 0 for r in rows]}, "ms",
              annotate=[f"{r.get('speedup', 0):.1f}x" for r in rows])  # fmt: skip
        ax.set_title(f"modules at {first.get('tokens')} tokens ({'forward + backward' if first.get('backward') else 'forward'})")
    elif "regime" in first:  # bench_pairformer_stack
        keys = sorted({(r["regime"], r["tokens"]) for r in rows})
        labels = [f"{reg} {tok}" for reg, tok in keys]
        series = {}
        for impl in sorted({r["impl"] for r in rows}):
            lookup = {(r["regime"], r["tokens"]): r["ms"] for r in rows if r["impl"] == impl}
            series[impl] = [lookup.get(k, 0) for k in keys]
        _bars(ax, labels, series, "ms")
        ax.set_title(f"{first.get('blocks')} Pairformer blocks")
    elif "out_err_kernels" in first:  # verify
        labels = [r["module"] for r in rows]
        _bars(ax, labels, {"kernels, output": [r["out_err_kernels"] for r in rows], "PyTorch bf16, output": [r["out_err_pytorch_bf16"] for r in rows],
                           "kernels, gradient": [r["grad_err_kernels"] for r in rows], "PyTorch bf16, gradient": [r["grad_err_pytorch_bf16"] for r in rows]},
              "relative error against fp32", log=True)  # fmt: skip
    else:
        raise ValueError(f"{path}: rows of an unknown benchmark")
    fig.tight_layout()
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, os.path.splitext(os.path.basename(path))[0] + ".png")
    fig.savefig(out, dpi=130)
    plt.close(fig)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("files", nargs="+")
    ap.add_argument("--out", default="plots")
    args = ap.parse_args(argv)
    for path in args.files:
        print(plot_file(path, args.out))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
