"""Time the real training input pipeline before a long run.

    python deploy/slurm/smoke_data.py --config configs/initial.yaml --dataset pdb:/data/pdb --examples 64

Builds exactly the stream the ``train`` command builds (datasets, weighted cluster sampling, mixture, cropping, MSA
loading, token-budget batching, prefetch thread), pulls ``--examples`` batches from it on the CPU and prints examples
per second, the slowest example, the feature shapes of the first batch and the stream's own counters (retries,
skipped records). A step of the model at crop 384 takes about 0.9 s on a B200, so one rank needs a little over one
example per second; ``--min-rate`` turns that into an exit code. The reference's pre-flight does the same with its
DataLoader (hangang/smoke_data.py).
"""

from __future__ import annotations

import argparse
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", action="append", default=[])
    ap.add_argument("--override", action="append", default=[])
    ap.add_argument("--dataset", action="append", default=[], help="name:path[:weight[:strategy[:distill]]]")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--examples", type=int, default=32)
    ap.add_argument("--num-workers", type=int, default=None)
    ap.add_argument("--min-rate", type=float, default=0.0, help="fail below this many examples per second")
    args = ap.parse_args(argv)

    import torch

    from deepfold3_dev_b200.cli.main import build_training_stream
    from deepfold3_dev_b200.config.loader import build_configs
    from deepfold3_dev_b200.parallel.dist import DistInfo

    tc, mc = build_configs(args.config, args.override)
    info = DistInfo()  # one rank's share of the data; the sampler strides by rank exactly as in training
    t0 = time.perf_counter()
    stream, _ = build_training_stream(tc, mc, info, args.dataset, None, args.synthetic, args.num_workers)
    print(f"stream built in {time.perf_counter() - t0:.1f} s")

    it = iter(stream)
    times, first = [], None
    for k in range(args.examples):
        t = time.perf_counter()
        batch = next(it)
        times.append(time.perf_counter() - t)
        if first is None:
            first = batch
            print(f"first batch after {times[0]:.2f} s")
    feats = first[0] if isinstance(first, (list, tuple)) else first
    for key in sorted(feats)[:400]:
        v = feats[key]
        if torch.is_tensor(v):
            print(f"  {key:36s} {tuple(v.shape)!s:24s} {str(v.dtype).replace('torch.', '')}")
    steady = times[1:] or times
    rate = len(steady) / max(sum(steady), 1e-9)
    print(f"{len(times)} batches: {rate:.2f} per second after the first, slowest {max(steady):.2f} s")
    counters = getattr(stream, "counters", None)
    if callable(counters):
        print("counters:", counters())
    if args.min_rate and rate < args.min_rate:
        print(f"FAIL: {rate:.2f} < {args.min_rate} batches per second")
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
