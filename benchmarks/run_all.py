#!/usr/bin/env python
"""Run every benchmark of this directory plus the kernel microbenchmarks and collect their output under one folder.

    python benchmarks/run_all.py [--out bench_results] [--skip inference]

Counterpart of the reference's benchmarks/run_all.py. Each step runs as its own process; a failing step is recorded and
the rest still run. ``summary.json`` lists the steps with their exit codes and wall times.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STEPS = {
    "kernels": [sys.executable, "-m", "deepfold3_dev_b200.ops.microbench", "--op", "all"],
    "modules_forward": [sys.executable, "benchmarks/bench_modules.py", "--json", "{out}/modules_forward.json"],
    "modules_backward": [sys.executable, "benchmarks/bench_modules.py", "--backward", "--json", "{out}/modules_backward.json"],
    "memory_inference": [sys.executable, "benchmarks/profile_memory.py", "--mode", "inference"],
    "memory_train": [sys.executable, "benchmarks/profile_memory.py", "--mode", "train", "--tokens", "128", "256", "384"],
    "verify": [sys.executable, "benchmarks/verify.py", "--json", "{out}/verify.json"],
    "pairformer_stack": [sys.executable, "benchmarks/bench_pairformer_stack.py", "--json", "{out}/pairformer_stack.json"],
    "complexlm": [sys.executable, "benchmarks/bench_complexlm.py"],
    "inference": [sys.executable, "benchmarks/bench_inference.py"],
    "train_step": [sys.executable, "bench.py", "--steps", "5", "--warmup", "3"],
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="bench_results")
    ap.add_argument("--skip", nargs="*", default=[], choices=list(STEPS))
    ap.add_argument("--only", nargs="*", default=None, choices=list(STEPS))
    args = ap.parse_args()
    out = os.path.abspath(args.out)
    os.makedirs(out, exist_ok=True)
    summary = []
    for name, cmd in STEPS.items():
        if name in args.skip or (args.only is not None and name not in args.only):
            continue
        cmd = [c.format(out=out) for c in cmd]
        t0 = time.time()
        with open(os.path.join(out, f"{name}.log"), "w") as log:
            rc = subprocess.run(cmd, cwd=ROOT, stdout=log, stderr=subprocess.STDOUT).returncode
        summary.append({"step": name, "returncode": rc, "seconds": round(time.time() - t0, 1), "command": " ".join(cmd)})
        print(json.dumps(summary[-1]), flush=True)
    with open(os.path.join(out, "summary.json"), "w") as f:
        json.dump(summary, f, indent=1)
    if any(s["returncode"] for s in summary):
        raise SystemExit(1)


if __name__ == "__main__":
    main()
