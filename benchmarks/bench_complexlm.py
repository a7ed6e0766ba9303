#!/usr/bin/env python
"""Training step of the complex language model at the shape the reference publishes a B200 figure for.

    python benchmarks/bench_complexlm.py                         # configs/plm-base.yaml, 16384 tokens per step
    python benchmarks/bench_complexlm.py --token-budget 32768 --steps 5

The reference reports for its 672 M-parameter model (33 layers x 1280, 20 heads, alternating chain-scoped and
complex-scoped layers) on one B200 at a token budget of 16384: 267 ms per step, 59k tokens per second, 52.6 GiB
(docs/complex-lm.md:48-49). This script builds the same model from ``configs/plm-base.yaml``, packs synthetic
two-chain complexes (random residues, 15 % masked) up to the token budget and times the trainer's own ``train_step``
(forward, loss, backward, clipping, fused AdamW) with CUDA events after warm-up, an L2 flush between steps; the end-to-end
figure copies the packed batch from pinned host memory inside the timed region and reads the loss back.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

PUBLISHED = {"ms_per_step": 267.0, "tokens_per_s": 59_000.0, "peak_gib": 52.6, "token_budget": 16384}


def synthetic_batch(token_budget: int, chain_len: int, seed: int):
    import numpy as np

    from deepfold3_dev_b200.complexlm.data import Example, pack
    from deepfold3_dev_b200.complexlm.model import IGNORE_INDEX, MASK_ID

    rng = np.random.default_rng(seed)
    examples, used = [], 0
    while used + 2 * chain_len <= token_budget:
        chains = [rng.integers(4, 24, size=chain_len), rng.integers(4, 24, size=chain_len)]
        toks, labels = [], []
        for c in chains:
            masked = rng.random(chain_len) < 0.15
            toks.append(np.where(masked, MASK_ID, c))
            labels.append(np.where(masked, c, IGNORE_INDEX))
        examples.append(Example(toks, labels, [0, 0], np.array([0, 1]), [np.zeros(chain_len, bool)] * 2, False, 0))
        used += 2 * chain_len
    return pack(examples)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default=os.path.join(ROOT, "configs", "plm-base.yaml"))
    ap.add_argument("--token-budget", type=int, default=16384)
    ap.add_argument("--chain-len", type=int, default=512)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)

    import torch

    from deepfold3_dev_b200.complexlm.config import load_experiment
    from deepfold3_dev_b200.complexlm.trainer import ComplexLMTrainer

    cfg = load_experiment(args.config, {"data.token_budget": args.token_budget})
    cfg.data.sources, cfg.eval_sources = [], []  # synthetic batches: no store on disk
    with tempfile.TemporaryDirectory() as out:
        trainer = ComplexLMTrainer(cfg, out)
        n_params = sum(p.numel() for p in trainer.model.parameters())
        batches = [synthetic_batch(args.token_budget, args.chain_len, s) for s in range(4)]
        for b in batches:  # pinned host copies, moved to the device inside the timed region of the end-to-end figure
            for name, v in vars(b).items():
                if torch.is_tensor(v):
                    setattr(b, name, v.pin_memory())
        tokens = batches[0].n_tokens
        flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        dev_batches = [b.to(trainer.device) for b in batches]

        def timed(get_batch, read_loss: bool) -> float:
            for i in range(args.warmup):
                trainer.train_step([get_batch(i)])
            times = []
            for i in range(args.steps):
                flush.zero_()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                out_metrics = trainer.train_step([get_batch(i)])
                if read_loss:
                    float(out_metrics["loss"])
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b))
            return sum(times) / len(times)

        torch.cuda.reset_peak_memory_stats()
        ms = timed(lambda i: dev_batches[i % 4], False)
        e2e = timed(lambda i: batches[i % 4], True)
        h2d = sum(v.numel() * v.element_size() for v in vars(batches[0]).values() if torch.is_tensor(v))
        row = {"metric": "complexlm train step", "model_params": n_params, "tokens_per_step": tokens, "ms_per_step": round(ms, 2),
               "tokens_per_s": round(tokens / ms * 1e3), "peak_gib": round(torch.cuda.max_memory_allocated() / 2**30, 1),
               "e2e": {"ms_per_step": round(e2e, 2), "tokens_per_s": round(tokens / e2e * 1e3), "h2d_bytes_per_step": h2d,
                       "d2h_bytes_per_step": 12},
               "dtype": cfg.train.dtype, "steps": args.steps, "warmup": args.warmup,
               "published_b200": PUBLISHED if args.token_budget == PUBLISHED["token_budget"] else None}  # fmt: skip
        if row["published_b200"]:
            row["x_vs_published"] = round(PUBLISHED["ms_per_step"] / ms, 2)
        from deepfold3_dev_b200.ops import autograd_ops

        autograd_ops.check_status()  # a kernel wait that ran out would make the figure meaningless: fail instead
        print(json.dumps(row), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
