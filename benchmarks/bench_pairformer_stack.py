#!/usr/bin/env python
"""A stack of Pairformer blocks at trunk shapes: inference forward and training forward+backward.

    python benchmarks/bench_pairformer_stack.py                          # 8 blocks, N = 384 640 768, both regimes
    python benchmarks/bench_pairformer_stack.py --impl reference         # the reference's blocks, its fused flags on
    python benchmarks/bench_pairformer_stack.py --regime inference --tokens 384 --json out.json

The one micro-benchmark the reference publishes for a B200 (docs/optimizations.md:22-49, measured with its
scripts/bench_kernels.py): 8 ``PairFormerBlock`` (pair 128 channels, single 384), batch 1, bf16 autocast, all-ones
masks; inference = forward under ``no_grad``; training = forward + backward of ``mean(pair^2) + mean(single^2)`` with
every block under activation checkpointing. Its published figures are in ``PUBLISHED`` below and are printed next to
what is measured here. Timing here: CUDA events on the launching stream, warm-up, a 256 MB write between runs to flush
L2, median; the reference's script times with the host clock around a synchronize, which for runs of tens of
milliseconds gives the same figure.

``--impl reference`` builds the same stack out of the reference package installed under ``baseline/_ref`` (its own
``PairFormerBlock`` with all four optional fused flags on, the configuration of its best published row) and times it
with the same harness, so both arms can be taken on one box.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

C_PAIR, C_SINGLE = 128, 384
# B200, 8 blocks (reference: docs/optimizations.md:22-49). ms for inference; training is published only relative to
# its own baseline, so the absolute training figure of the reference comes from --impl reference.
PUBLISHED = {
    "inference_ms": {"baseline": {384: 52.98, 640: 164.85, 768: 257.34}, "all_four_fused": {384: 35.58, 640: 114.78, 768: 173.46}},
    "inference_peak_gb": {"baseline": {384: 0.9, 640: 2.4, 768: 3.4}, "all_four_fused": {384: 0.7, 640: 1.9, 768: 2.7}},
    "training_peak_gb": {"baseline": {384: 3.18, 640: 8.72, 768: 12.52}},
    "training_speedup_all_four": {384: 1.01, 640: 1.17, 768: 1.25},
}


def gpu_time(fn, warmup: int, iters: int) -> float:
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


def build_blocks(impl: str, n_blocks: int):
    import torch

    if impl == "ours":
        from deepfold3_dev_b200.models.evoformer import PairFormerBlock

        blocks = [PairFormerBlock(C_PAIR, C_SINGLE) for _ in range(n_blocks)]
    else:
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm

        sys.path.insert(0, reference_arm.REF_PATH)
        reference_arm._stub_missing()
        from deepfold3.model.config import OptimConfig
        from deepfold3.model.evoformer import PairFormerBlock

        optim = OptimConfig()
        for flag in ("use_fused_evo_attention", "use_fused_dropout_add", "use_fused_swiglu", "use_fused_transition_pair",
                     "use_fused_triangle_mul", "use_fused_pair_bias"):  # fmt: skip
            setattr(optim, flag, True)
        blocks = [PairFormerBlock(c_pair=C_PAIR, c_single=C_SINGLE, optim=optim) for _ in range(n_blocks)]
    return torch.nn.ModuleList(blocks).cuda().to(torch.bfloat16)


def run(blocks, pair, single, pair_mask, seq_mask, checkpoint: bool):
    import torch
    from torch.utils.checkpoint import checkpoint as ckpt

    for blk in blocks:
        if checkpoint and torch.is_grad_enabled():
            pair, single = ckpt(blk, pair, single, pair_mask, seq_mask, use_reentrant=False)
        else:
            pair, single = blk(pair, single, pair_mask, seq_mask)
    return pair, single


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--blocks", type=int, default=8)
    ap.add_argument("--tokens", type=int, nargs="+", default=[384, 640, 768])
    ap.add_argument("--regime", choices=["inference", "training", "both"], default="both")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--json", type=str, default=None)
    args = ap.parse_args(argv)

    import torch

    torch.manual_seed(0)
    blocks = build_blocks(args.impl, args.blocks)
    rows = []
    for n in args.tokens:
        g = torch.Generator(device="cuda").manual_seed(0)
        pair0 = torch.randn(1, n, n, C_PAIR, device="cuda", dtype=torch.bfloat16, generator=g)
        single0 = torch.randn(1, n, C_SINGLE, device="cuda", dtype=torch.bfloat16, generator=g)
        pair_mask = torch.ones(1, n, n, device="cuda", dtype=torch.bfloat16)
        seq_mask = torch.ones(1, n, device="cuda", dtype=torch.bfloat16)
        if args.regime in ("inference", "both"):
            blocks.eval()

            def infer():
                with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                    run(blocks, pair0, single0, pair_mask, seq_mask, False)

            infer()
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            ms = gpu_time(infer, args.warmup, args.iters)
            row = {"impl": args.impl, "regime": "inference", "blocks": args.blocks, "tokens": n, "ms": round(ms, 3),
                   "peak_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2)}  # fmt: skip
            if args.blocks == 8 and n in PUBLISHED["inference_ms"]["baseline"]:
                row["published_ms_baseline"] = PUBLISHED["inference_ms"]["baseline"][n]
                row["published_ms_all_four_fused"] = PUBLISHED["inference_ms"]["all_four_fused"][n]
                row["x_vs_published_best"] = round(PUBLISHED["inference_ms"]["all_four_fused"][n] / ms, 2)
            rows.append(row)
            print(json.dumps(row), flush=True)
        if args.regime in ("training", "both"):
            blocks.train()
            pair = pair0.clone().requires_grad_(True)
            single = single0.clone().requires_grad_(True)

            def train():
                for p in blocks.parameters():
                    p.grad = None
                pair.grad = single.grad = None
                with torch.autocast("cuda", dtype=torch.bfloat16):
                    op, os_ = run(blocks, pair, single, pair_mask, seq_mask, True)
                    loss = op.float().pow(2).mean() + os_.float().pow(2).mean()
                loss.backward()

            train()
            torch.cuda.synchronize()
            torch.cuda.reset_peak_memory_stats()
            ms = gpu_time(train, args.warmup, args.iters)
            row = {"impl": args.impl, "regime": "training_ckpt", "blocks": args.blocks, "tokens": n, "ms": round(ms, 3),
                   "peak_gb": round(torch.cuda.max_memory_allocated() / 2**30, 2)}  # fmt: skip
            if args.blocks == 8 and n in PUBLISHED["training_peak_gb"]["baseline"]:
                row["published_peak_gb_baseline"] = PUBLISHED["training_peak_gb"]["baseline"][n]
            rows.append(row)
            print(json.dumps(row), flush=True)
    if args.impl == "ours":
        from deepfold3_dev_b200.ops.autograd_ops import check_status

        check_status()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
