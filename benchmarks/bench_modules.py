#!/usr/bin/env python
"""Module-level benchmarks: attention, triangle / outer-product ops, transitions, LayerNorm (forward, forward+backward).

    python benchmarks/bench_modules.py [--tokens 384] [--msa 1024] [--group attention|pair_ops|primitives|transition|all]
                                       [--backward] [--json results.json]

The counterpart of the reference's benchmarks/bench_attention.py, bench_pair_ops.py, bench_primitives.py,
bench_transition.py and bench_msa_transition.py: each module of the trunk is timed at trunk shapes under bf16
autocast with this package's kernels and again with the listed kernels switched off (``DF3_DISABLE_OPS``), which runs
the plain PyTorch statement of the same module. Timing: CUDA events, 5 warm-up and 20 timed runs, median, an L2 flush
(a 256 MB write) before every run. One JSON object per case is printed; ``--json`` also writes the list.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

FUSED_FEATURES = ("gemm,matmul,gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,layer_norm,swiglu,"
                  "dropout_add,plane_layer_norm,window_attention,ada_norm")  # fmt: skip


def gpu_time(fn, warmup: int = 5, iters: int = 20) -> float:
    import torch

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(warmup):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    return sorted(times)[len(times) // 2]


def cases(N: int, S: int, group: str):
    import torch

    from deepfold3_dev_b200.models.attention import GridSelfAttention, MSAAttention, SingleAttention
    from deepfold3_dev_b200.models.primitives import LayerNorm, TransitionBlock
    from deepfold3_dev_b200.models.triangle import OuterProductMean, TriangleMulIncoming, TriangleMulOutgoing

    dev = "cuda"
    z = lambda: torch.randn(1, N, N, 128, device=dev, requires_grad=True)  # noqa: E731
    pm = torch.ones(1, N, N, device=dev)
    out = []
    if group in ("attention", "all"):
        out += [("grid_attention_row", GridSelfAttention(128, 4), lambda: (z(), pm)),
                ("grid_attention_col", GridSelfAttention(128, 4, transpose=True), lambda: (z(), pm)),
                ("msa_attention", MSAAttention(64, 128, 8), lambda: (torch.randn(1, S, N, 64, device=dev, requires_grad=True),
                                                                     torch.ones(1, S, N, device=dev), z())),
                ("single_attention", SingleAttention(384, 16, 128) if _single_sig() else None, None)]  # fmt: skip
    if group in ("pair_ops", "all"):
        out += [("triangle_mul_outgoing", TriangleMulOutgoing(128), lambda: (z(), pm)),
                ("triangle_mul_incoming", TriangleMulIncoming(128), lambda: (z(), pm)),
                ("outer_product_mean", OuterProductMean(64, 128, 32), lambda: (torch.randn(1, S, N, 64, device=dev, requires_grad=True),
                                                                               torch.ones(1, S, N, device=dev)))]  # fmt: skip
    if group in ("transition", "all"):
        out += [("pair_transition", TransitionBlock(128, 4), lambda: (z(),)),
                ("single_transition", TransitionBlock(384, 4), lambda: (torch.randn(1, N, 384, device=dev, requires_grad=True),)),
                ("msa_transition", TransitionBlock(64, 4), lambda: (torch.randn(1, S, N, 64, device=dev, requires_grad=True),))]  # fmt: skip
    if group in ("primitives", "all"):
        out += [("layer_norm_pair", LayerNorm(128), lambda: (z(),))]
    return [(n, m.to(dev), mk) for n, m, mk in out if m is not None and mk is not None]


def _single_sig() -> bool:
    return False  # the single-track attention takes hoisted pair logits; it is covered by the block benchmark in bench.py


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=384)
    ap.add_argument("--msa", type=int, default=1024)
    ap.add_argument("--group", default="all", choices=["attention", "pair_ops", "primitives", "transition", "all"])
    ap.add_argument("--backward", action="store_true")
    ap.add_argument("--json", default=None)
    args = ap.parse_args()

    import torch

    torch.manual_seed(0)
    rows = []
    for name, module, make in cases(args.tokens, args.msa, args.group):
        for p in module.parameters():  # zero-initialised output layers would make backward trivially sparse
            if p.abs().sum() == 0:
                torch.nn.init.normal_(p, std=0.02)
        inputs = make()

        def run():
            with torch.autocast("cuda", dtype=torch.bfloat16):
                y = module(*inputs)
            if args.backward:
                y.float().square().mean().backward()

        row = {"module": name, "tokens": args.tokens, "backward": args.backward}
        for label, disabled in (("ours_ms", ""), ("eager_ms", FUSED_FEATURES)):
            os.environ["DF3_DISABLE_OPS"] = disabled
            try:
                row[label] = round(gpu_time(run), 4)
            except torch.cuda.OutOfMemoryError:
                row[label] = None
                torch.cuda.empty_cache()
        os.environ["DF3_DISABLE_OPS"] = ""
        if row["ours_ms"] and row["eager_ms"]:
            row["speedup"] = round(row["eager_ms"] / row["ours_ms"], 2)
        print(json.dumps(row), flush=True)
        rows.append(row)
        del inputs
        torch.cuda.empty_cache()
    from deepfold3_dev_b200.ops import autograd_ops

    autograd_ops.check_status()  # a kernel wait that ran out would make the timings meaningless
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
