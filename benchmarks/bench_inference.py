#!/usr/bin/env python
"""Inference benchmark: seconds per prediction (trunk with recycling + diffusion samples + confidence head).

    python benchmarks/bench_inference.py --tokens 1024 --samples 5 --recycles 10 --steps 200 [--impl ours|reference]

Default config is the second headline metric: N = 1024 tokens (3 protein chains + one 30-atom ligand), 5 samples,
10 recycles, 200 sampler steps, 4096 MSA rows, no templates, bf16 autocast, random-init weights, synthetic features
(the same job as ``bench.py --config infer1024``, which also runs it on several GPUs and reports end-to-end time).
One untimed prediction warms kernels and (for this package) captures the sampler's CUDA graph; then
``--repeats`` predictions are timed with CUDA events and the median is reported on one JSON line.
``--impl reference`` runs the unmodified reference package from ``baseline/_ref`` with its ``inference``
kernel preset on the same features.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=1024)
    ap.add_argument("--chains", type=int, default=3, help="protein chains")
    ap.add_argument("--ligand-atoms", type=int, default=30, help="atoms of the one ligand chain (0: no ligand)")
    ap.add_argument("--samples", type=int, default=5)
    ap.add_argument("--recycles", type=int, default=10)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--msa", type=int, default=4096)
    ap.add_argument("--templates", type=int, default=0)
    ap.add_argument("--repeats", type=int, default=2)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()

    import torch

    from deepfold3_dev_b200.data.synthetic import split_lengths, synthetic_complex

    dev = torch.device("cuda", 0)
    chains = [("protein", n) for n in split_lengths(args.tokens - args.ligand_atoms, args.chains)]
    if args.ligand_atoms:
        chains.append(("ligand", args.ligand_atoms))
    feats = synthetic_complex(chains, num_msa=args.msa, num_templates=args.templates, seed=11, with_gt=False)
    feats = {k: v.to(dev) for k, v in feats.items()}
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        from baseline.reference_arm import _stub_missing

        _stub_missing()
        try:
            from deepfold3.model.config import ModelConfig, OptimConfig
            from deepfold3.model.model import DeepFold3
        except Exception as exc:  # noqa: BLE001
            print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {exc}"[:300]}))
            return
        cfg = ModelConfig()
        cfg.optim = OptimConfig.inference()
    else:
        from deepfold3_dev_b200.config.schema import ModelConfig, OptimConfig
        from deepfold3_dev_b200.models.model import DeepFold3

        cfg = ModelConfig()
        cfg.optim = OptimConfig.inference()
    cfg.msa_crop_size = args.msa
    cfg.diffusion.steps = args.steps
    cfg.diffusion.num_samples = args.samples
    torch.manual_seed(0)
    model = DeepFold3(cfg).to(dev).eval()

    def predict(seed):
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(dict(feats), seed=seed, num_recycles=args.recycles, num_samples=args.samples)
        return out.atom_positions.float().abs().mean().item()  # device -> host read of the result

    predict(0)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    times = []
    for r in range(args.repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        predict(1 + r)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) / 1e3)
    times.sort()
    if args.impl == "ours":
        from deepfold3_dev_b200.ops import autograd_ops

        autograd_ops.check_status()  # a kernel wait that ran out would make the timings meaningless
    print(json.dumps({
        "metric": "inference seconds per prediction", "value": times[len(times) // 2], "unit": "s", "higher_is_better": False,
        "impl": args.impl, "dtype": "bf16", "data": "synthetic (random sequences, random-init weights)",
        "config": {"tokens": args.tokens, "chains": args.chains, "ligand_atoms": args.ligand_atoms, "samples": args.samples, "recycles": args.recycles,
                   "sampler_steps": args.steps, "msa_rows": args.msa, "templates": args.templates,
                   "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2**30, 2)},
        "all_s": times,
    }))  # fmt: skip


if __name__ == "__main__":
    main()
