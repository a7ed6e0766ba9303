#!/usr/bin/env python
"""Peak device memory of inference and of one training step as a function of the token count.

    python benchmarks/profile_memory.py [--mode inference|train] [--tokens 256 384 512 768 1024] [--limit-gib 150]

The counterpart of the reference's benchmarks/profile_memory.py. Each size runs in this process after
``torch.cuda.reset_peak_memory_stats``; a size whose predicted footprint (quadratic fit through the previous points)
exceeds ``--limit-gib`` is skipped rather than attempted, so the sweep never drives the device out of memory.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def predicted_gib(points: list[tuple[int, float]], n: int) -> float:
    """Quadratic extrapolation a + b n^2 through the last two measurements (pair activations dominate)."""
    if len(points) < 2:
        return 0.0
    (n0, m0), (n1, m1) = points[-2], points[-1]
    b = (m1 - m0) / max(n1 * n1 - n0 * n0, 1)
    return m1 + b * (n * n - n1 * n1)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", default="inference", choices=["inference", "train"])
    ap.add_argument("--tokens", type=int, nargs="+", default=[256, 384, 512, 768, 1024])
    ap.add_argument("--msa", type=int, default=1024)
    ap.add_argument("--limit-gib", type=float, default=150.0)
    args = ap.parse_args()

    import torch

    from deepfold3_dev_b200.config.schema import ModelConfig, TrainingConfig
    from deepfold3_dev_b200.data.datasets import collate
    from deepfold3_dev_b200.data.synthetic import synthetic_complex, split_lengths
    from deepfold3_dev_b200.models.model import DeepFold3

    dev = torch.device("cuda")
    cfg = ModelConfig()
    cfg.msa_crop_size = args.msa
    cfg.diffusion.steps = 4  # the footprint does not depend on the number of sampler steps
    model = DeepFold3(cfg).to(dev)
    points: list[tuple[int, float]] = []
    for n in sorted(args.tokens):
        guess = predicted_gib(points, n)
        if guess > args.limit_gib:
            print(json.dumps({"tokens": n, "skipped": f"predicted {guess:.0f} GiB > limit {args.limit_gib:.0f} GiB"}))
            continue
        feats = synthetic_complex([("protein", m) for m in split_lengths(n, 2)], num_msa=args.msa, num_templates=4, seed=0,
                                  with_gt=args.mode == "train")
        if args.mode == "train":
            batch = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in collate([feats]).items()}
        else:
            batch = {k: v.to(dev) for k, v in feats.items()}
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
        if args.mode == "inference":
            model.eval()
            with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
                model(dict(batch), seed=0, num_recycles=1, num_samples=1)
        else:
            from deepfold3_dev_b200.training.engine import training_step

            model.train()
            tc = TrainingConfig(max_tokens=n)
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss, *_ = training_step(model, batch, cfg=tc, model_cfg=cfg, global_step=0, device=dev, num_recycles=1)
            loss.backward()
            model.zero_grad(set_to_none=True)
        torch.cuda.synchronize()
        gib = torch.cuda.max_memory_allocated() / 2**30
        points.append((n, gib))
        print(json.dumps({"tokens": n, "mode": args.mode, "peak_gib": round(gib, 2)}), flush=True)


if __name__ == "__main__":
    main()
