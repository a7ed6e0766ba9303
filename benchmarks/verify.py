#!/usr/bin/env python
"""Numerical check of every trunk module: this package's kernels against the PyTorch statement of the same module.

    python benchmarks/verify.py [--tokens 256] [--msa 256] [--group all] [--json verify.json]

For each module of ``bench_modules.cases`` the same weights and inputs run twice under bf16 autocast: with the kernels,
and with the listed kernels switched off (``DF3_DISABLE_OPS``), which is the plain PyTorch bf16 path; a third run in fp32
without autocast is the oracle. Reported per module: the largest absolute error of the output and of the input gradient
for both bf16 paths against the fp32 oracle, relative to the oracle's largest magnitude. A module passes when the
kernel path's error is at most ``--slack`` (default 2) times the PyTorch bf16 path's, or below ``--floor``. Exit code 1
on any failure. Counterpart of the reference's benchmarks/verify.py (fused Triton paths against its stock modules).
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--msa", type=int, default=256)
    ap.add_argument("--group", default="all", choices=["attention", "pair_ops", "primitives", "transition", "all"])
    ap.add_argument("--slack", type=float, default=2.0)
    ap.add_argument("--floor", type=float, default=2e-2)
    ap.add_argument("--json", default=None)
    args = ap.parse_args(argv)

    import torch

    import bench_modules

    torch.manual_seed(0)
    rows, failed = [], 0
    for name, module, make in bench_modules.cases(args.tokens, args.msa, args.group):
        for p in module.parameters():
            if p.abs().sum() == 0:
                torch.nn.init.normal_(p, std=0.02)
        inputs = make()
        weight = None

        def run(autocast: bool, disabled: str):
            nonlocal weight
            os.environ["DF3_DISABLE_OPS"] = disabled
            try:
                leaves = [t.detach().clone().requires_grad_(t.requires_grad) for t in inputs]
                with torch.autocast("cuda", dtype=torch.bfloat16, enabled=autocast):
                    y = module(*leaves)
                if weight is None:
                    weight = torch.randn_like(y.float())
                (y.float() * weight).sum().backward()
                grad = next((t.grad.float() for t in leaves if t.grad is not None), None)
                for p in module.parameters():
                    p.grad = None
                return y.detach().float(), grad
            finally:
                os.environ["DF3_DISABLE_OPS"] = ""

        oracle_y, oracle_g = run(False, bench_modules.FUSED_FEATURES)
        ours_y, ours_g = run(True, "")
        eager_y, eager_g = run(True, bench_modules.FUSED_FEATURES)

        def err(a, b):
            return float((a - b).abs().max() / b.abs().max().clamp(min=1e-12)) if a is not None and b is not None else 0.0

        row = {"module": name, "tokens": args.tokens, "out_err_kernels": err(ours_y, oracle_y), "out_err_pytorch_bf16": err(eager_y, oracle_y),
               "grad_err_kernels": err(ours_g, oracle_g), "grad_err_pytorch_bf16": err(eager_g, oracle_g)}  # fmt: skip
        ok = all(row[f"{k}_err_kernels"] <= max(args.floor, args.slack * row[f"{k}_err_pytorch_bf16"]) for k in ("out", "grad"))
        row["pass"] = bool(ok)
        failed += not ok
        print(json.dumps(row), flush=True)
        rows.append(row)
        del inputs
        torch.cuda.empty_cache()
    from deepfold3_dev_b200.ops import autograd_ops

    autograd_ops.check_status()
    if args.json:
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)
    print(f"{len(rows) - failed} of {len(rows)} modules within tolerance")
    return 1 if failed else 0


if __name__ == "__main__":
    raise SystemExit(main())
