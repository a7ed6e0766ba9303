#!/usr/bin/env python
"""Where the time of one training step goes: phase split by CUDA events, kernel table and Chrome trace by torch.profiler.

    python benchmarks/profile_training.py                                   # crop 384, full model, phase split only
    python benchmarks/profile_training.py --table 40 --trace step.json      # + kernel shares and a trace for chrome://tracing
    python benchmarks/profile_training.py --tokens 768 --checkpointing --by-shape

The step is the one ``bench.py`` times (same synthetic example, same training settings, the trainer's own
``micro_step`` + optimizer step). Three views, each optional because each perturbs the step more than the one before:

* phase split (always): forward + loss / backward / optimizer, and inside the forward the trunk passes, the template
  embedding, the no-grad mini-rollout, the 48-sample diffusion forward and the confidence head, from CUDA events
  recorded around the calls of an otherwise unmodified step;
* ``--table N``: the N kernels and the N host-side operators with the largest totals (torch.profiler); a step whose
  host total exceeds its device total is launch-bound;
* ``--by-shape``: framework element-wise / copy / reduction operators grouped by input shape, which is how fusion
  candidates are found (the own kernels show up under their operator names in ``--table``);
* ``--trace FILE``: Chrome trace of one profiled step.

Set ``DF3_NVTX=1`` to get NVTX ranges around every kernel-op call for an external timeline tool. The reference has the
same tool for its trainer (scripts/profile_training.py:131-150, a torch.profiler wrapper around its step).
"""

from __future__ import annotations

import argparse
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--tokens", type=int, default=384)
    ap.add_argument("--recycles", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--checkpointing", action="store_true", help="Recompute the trunk blocks in backward.")
    ap.add_argument("--blocks", type=int, default=0, help="Pairformer depth (0: the model's 48).")
    ap.add_argument("--table", type=int, default=0, help="Rows of the kernel and host tables (0: skip the profiler).")
    ap.add_argument("--by-shape", action="store_true")
    ap.add_argument("--trace", type=str, default=None)
    args = ap.parse_args(argv)

    import torch
    from torch.profiler import ProfilerActivity, profile

    import bench
    from deepfold3_dev_b200.config.schema import ModelConfig, TrainingConfig
    from deepfold3_dev_b200.ops import autograd_ops
    from deepfold3_dev_b200.parallel.dist import DistInfo
    from deepfold3_dev_b200.training.engine import training_step
    from deepfold3_dev_b200.training.trainer import Trainer

    mc = ModelConfig()
    mc.msa_crop_size = bench.N_MSA
    mc.optim.use_gradient_checkpointing = args.checkpointing
    if args.blocks:
        mc.pairformer.num_layer = args.blocks
    os.environ.setdefault("DF3_DIFFUSION_CKPT", "0")
    tc = TrainingConfig(**bench.shared_train_settings(args.tokens), output_dir="/tmp/df3_profile")
    dev = torch.device("cuda", 0)
    trainer = Trainer(tc, mc, dist_info=DistInfo(device=dev))
    batch = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in bench.make_host_batch(0, args.tokens).items()}

    def step():
        trainer.micro_step(dict(batch), num_recycles=args.recycles)
        trainer.engine.step_or_skip(trainer.state)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()

    # ---- phase split: events around the calls of one step
    marks = []

    def timed(name, fn):
        def wrapper(*a, **k):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = fn(*a, **k)
            e.record()
            marks.append((name, s, e))
            return out

        return wrapper

    m = trainer.model
    saved = [(m, "run_evoformer"), (m.diffusion_head, "sample"), (m.diffusion_head, "sample_training"),
             (m.confidence_head, "forward"), (m.evoformer.template_embedding, "forward")]  # fmt: skip
    labels = ["trunk pass", "mini-rollout (no grad)", "diffusion forward", "confidence head", "  template embedding"]
    originals = [getattr(obj, name) for obj, name in saved]
    for (obj, name), label, fn in zip(saved, labels, originals):
        setattr(obj, name, timed(label, fn))
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    ev[0].record()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        loss, *_ = training_step(m, dict(batch), cfg=tc, model_cfg=mc, global_step=0, device=dev, num_recycles=args.recycles)
    ev[1].record()
    loss.backward()
    ev[2].record()
    trainer.engine.add_microstep_loss(loss)
    trainer.engine.step_or_skip(trainer.state)
    ev[3].record()
    torch.cuda.synchronize()
    for (obj, name), fn in zip(saved, originals):
        setattr(obj, name, fn)
    print(f"tokens {args.tokens}, recycles {args.recycles}, checkpointing {args.checkpointing}")
    print(f"forward + loss {ev[0].elapsed_time(ev[1]):8.1f} ms")
    for name, s, e in marks:
        print(f"    {name:26s} {s.elapsed_time(e):8.1f} ms")
    print(f"backward       {ev[1].elapsed_time(ev[2]):8.1f} ms")
    print(f"optimizer      {ev[2].elapsed_time(ev[3]):8.1f} ms")
    print(f"peak memory    {torch.cuda.max_memory_allocated() / 2**30:8.1f} GiB")

    # ---- profiler views
    if args.table or args.trace or args.by_shape:
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU], record_shapes=args.by_shape) as prof:
            step()
            torch.cuda.synchronize()
        if args.trace:
            prof.export_chrome_trace(args.trace)
            print(f"trace -> {args.trace}")
        if args.table:
            print(prof.key_averages().table(sort_by="cuda_time_total", row_limit=args.table, max_name_column_width=60))
            print(prof.key_averages().table(sort_by="self_cpu_time_total", row_limit=args.table, max_name_column_width=60))
        if args.by_shape:
            rows = [e for e in prof.key_averages(group_by_input_shape=True) if e.key.startswith("aten::") and e.self_device_time_total > 0]
            rows.sort(key=lambda e: -e.self_device_time_total)
            print("framework operators by input shape (device time)")
            for e in rows[:60]:
                print(f"  {e.key:22s} {e.self_device_time_total / 1e3:8.2f} ms  n={e.count:5d}  {str(e.input_shapes)[:140]}")
    autograd_ops.check_status()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
