#!/usr/bin/env python
"""Headline benchmark: full AF3-size DeepFold3 training throughput (samples/s) at crop 384.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--config train384|finetune768|infer1024|long3072]

Config (both arms): default ModelConfig (4 MSA blocks, 48 Pairformer blocks, 24-block diffusion
transformer, 4 confidence blocks), bf16 autocast with fp32 master weights, one synthetic 2-chain
protein complex of 384 tokens (~3000 atoms) per GPU, 1024 MSA rows at 30 % mutation, 4 templates,
48 diffusion samples, 20-step mini-rollout, gradient accumulation 1, AdamW + EMA 0.999. A step is
forward + loss + backward + gradient reduction + optimizer + EMA; the number of recycles of step i
is ``Random(seed + i).randint(0, 3)`` in both arms. Weak scaling: one example per GPU.

``--impl reference`` drives the unmodified reference package installed under ``baseline/_ref``
through its own ``training_step`` / ``WrappedOptimizer`` / DDP path and prints the same JSON line.

Other configs (``--config``), same JSON line:

``finetune768``  training at crop 768: two protein chains plus a 20-nucleotide RNA, 2048 MSA rows, activation
                 checkpointing on in both arms (the pair activations of 48 blocks do not fit otherwise).
``infer1024``    seconds per prediction: 3 protein chains + a 30-atom ligand (1024 tokens), 4096 MSA rows, no templates,
                 10 recycles, 200 sampler steps, 5 samples. On N GPUs one prediction is spread over the GPUs: the trunk
                 row-sharded, the samples dealt out (the reference arm gives each process a share of the samples).
``long3072``     seconds per prediction at 3072 tokens (6 chains of 512), 2048 MSA rows, 10 recycles, 1 sample; the pair
                 tensor row-sharded over the GPUs (the reference arm is its single-GPU chunked path).
A "step" of the inference configs is one whole prediction.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
SEED = 101
N_TOKENS, N_MSA, N_TEMPLATES, N_DIFFUSION = 384, 1024, 4, 48
BASELINE_VALUE = None  # no B200 number is published for this metric


def _chains(kind_lengths):
    return lambda: list(kind_lengths)


CONFIGS = {
    "train384": dict(kind="train", tokens=384, msa=1024, templates=4, metric="train samples/s @crop384",
                     chains=lambda t: [("protein", (t + 1) // 2), ("protein", t // 2)]),
    "finetune768": dict(kind="train", tokens=768, msa=2048, templates=4, metric="train samples/s @crop768", checkpointing=True,
                        chains=lambda t: [("protein", (t - 20 + 1) // 2), ("protein", (t - 20) // 2), ("rna", 20)]),
    "infer1024": dict(kind="infer", tokens=1024, msa=4096, templates=0, recycles=10, sampler_steps=200, samples=5,
                      metric="inference s/prediction N=1024, 5 samples",
                      chains=lambda t: [("protein", (t - 30 + 2) // 3), ("protein", (t - 30 + 1) // 3), ("protein", (t - 30) // 3),
                                        ("ligand", 30)]),
    "long3072": dict(kind="infer", tokens=3072, msa=2048, templates=0, recycles=10, sampler_steps=200, samples=1,
                     metric="inference s/prediction N=3072, 1 sample", chains=lambda t: [("protein", t // 6)] * 6),
}  # fmt: skip


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="train384", choices=sorted(CONFIGS))
    ap.add_argument("--tokens", type=int, default=0, help="override the config's token count (debugging)")
    ap.add_argument("--blocks", type=int, default=0, help="debug only: override the Pairformer depth")
    ap.add_argument("--recycles", type=int, default=-1, help="inference configs, debug only: override the recycle count")
    ap.add_argument("--sampler-steps", type=int, default=0, help="inference configs, debug only: override the sampler steps")
    args = ap.parse_args()
    args.cfg = dict(CONFIGS[args.config])
    args.tokens = args.tokens or args.cfg["tokens"]
    global N_MSA, N_TEMPLATES
    N_MSA, N_TEMPLATES = args.cfg["msa"], args.cfg["templates"]
    return args


class ClockSampler:
    """nvidia-smi SM clock / throttle-reason samples every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")  # fmt: skip

    def __init__(self, gpu_index: int):
        self.gpu, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)  # fmt: skip
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}  # fmt: skip


def recycles_for(step: int, max_recycles: int = 3) -> int:
    import random

    return random.Random(SEED + step).randint(0, max_recycles)


def make_host_batch(rank: int, tokens: int, chains=None):
    """One synthetic example (batch axis 1) in pinned host memory; the generator imports only torch + tables."""
    import torch

    from deepfold3_dev_b200.data.synthetic import batch_features, synthetic_complex

    chains = chains or CONFIGS["train384"]["chains"]
    feats = synthetic_complex(chains(tokens), num_msa=N_MSA, num_templates=N_TEMPLATES, seed=1000 + rank)
    batch = batch_features([feats])
    if torch.cuda.is_available():
        batch = {k: (v.pin_memory() if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
    return batch


def batch_bytes(batch) -> int:
    import torch

    return int(sum(v.numel() * v.element_size() for v in batch.values() if isinstance(v, torch.Tensor)))


def flush_l2(buf):
    buf.add_(1)  # touches 256 MB, more than the 126 MB L2


def timed_loop(step_fn, steps: int, first_step: int, dist_barrier, flush_buf):
    """K steps bracketed by barrier + synchronize, each timed with CUDA events; returns per-step ms."""
    import torch

    dist_barrier()
    torch.cuda.synchronize()
    times = []
    for i in range(steps):
        flush_l2(flush_buf)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step_fn(first_step + i)
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1))
    dist_barrier()
    torch.cuda.synchronize()
    return times


def reduce_max(value: float, world: int) -> float:
    if world <= 1:
        return value
    import torch
    import torch.distributed as dist

    t = torch.tensor([value], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def emit(args, impl, step_ms, e2e_ms, clocks, launches, bytes_in, extra_cfg):
    world = args.gpus
    value = world * 1000.0 / step_ms
    line = {
        "metric": args.cfg["metric"],
        "value": value,
        "unit": "samples/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": step_ms,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": (value / BASELINE_VALUE) if BASELINE_VALUE else None,
        "dtype": "bf16",
        "data": "synthetic (random sequences, random-init weights)",
        "impl": impl,
        "config": {
            "model": "DeepFold3 default ModelConfig (48 Pairformer, 24 diffusion blocks, 368M params)",
            "global_batch": world,
            "seq_len": args.tokens,
            "msa_rows": N_MSA,
            "templates": N_TEMPLATES,
            "diffusion_samples": N_DIFFUSION,
            "parallelism": f"dp{world}",
            "l2": "256 MB buffer rewritten between timed steps; activations exceed L2",
            **extra_cfg,
        },
        "clocks": clocks,
        "e2e": {"value": world * 1000.0 / e2e_ms, "unit": "samples/s", "h2d_bytes_per_step": bytes_in,
                "d2h_bytes_per_step": 8, "ms_per_step": e2e_ms},  # fmt: skip
        "gpu_launches": launches,
    }
    print(json.dumps(line), flush=True)


def shared_train_settings(tokens: int) -> dict:
    """TrainingConfig fields set identically in both arms."""
    return dict(
        lr=1.8e-3, weight_decay=0.0, betas=(0.9, 0.95), eps=1e-8, warmup_steps=1000, grad_clip_norm=10.0,
        grad_norm_fp64=True, accumulate_grad_batches=1, ema_decay=0.999, max_tokens=tokens, max_atoms=4096,
        max_recycles=3, batch_size_per_rank=1, diffusion_batch_size=N_DIFFUSION, mini_rollout_steps=20,
        mini_rollout_samples=1, permute_gt_before_noise=True, alpha_diffusion=4.0, alpha_smooth_lddt=1.0,
        alpha_distogram=0.03, alpha_confidence=1e-4, alpha_pae=1.0, dtype="bf16", seed=SEED, uniform_recycle=True,
        log_tm_true=True, max_consecutive_nan_skips=100,
    )  # fmt: skip


def _graph_state(model) -> str:
    cache = model.__dict__.get("_trunk_train_graphs")
    if cache is None:
        return "off"
    return "failed, ran eagerly" if cache.failed else "forward + backward replayed from CUDA graphs"


def run_ours(args):
    import torch

    sys.path.insert(0, ROOT)
    from deepfold3_dev_b200.config.schema import ModelConfig, TrainingConfig
    from deepfold3_dev_b200.ops import autograd_ops
    from deepfold3_dev_b200.parallel.dist import barrier, init_process_group
    from deepfold3_dev_b200.training.trainer import Trainer

    info = init_process_group(timeout_s=1800.0)
    world = info.world_size
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    host_batch = make_host_batch(info.rank, args.tokens, args.cfg["chains"])
    dev_batch = {k: (v.to(info.device) if isinstance(v, torch.Tensor) else v) for k, v in host_batch.items()}
    flush_buf = torch.zeros(64 * 1024 * 1024, device=info.device)
    # Memory policies (trunk checkpointing, denoiser checkpointing, diffusion chunk), fastest first; one that runs out of
    # memory during warm-up is torn down and the next is built (all ranks move together). Crop 384 keeps everything
    # resident; crop 768 recomputes the trunk and tries to keep the denoiser's activations before giving that up too.
    # DF3_CKPT / DF3_DIFFUSION_CKPT / DF3_DIFFUSION_CHUNK pin one policy.
    if args.cfg.get("checkpointing"):
        ladder = [(True, False, 0), (True, True, 8)]
    else:
        ladder = [(False, False, 0)]
    if any(k in os.environ for k in ("DF3_CKPT", "DF3_DIFFUSION_CKPT", "DF3_DIFFUSION_CHUNK")):
        first = ladder[0]
        ladder = [(os.environ.get("DF3_CKPT", "1" if first[0] else "0") == "1",
                   os.environ.get("DF3_DIFFUSION_CKPT", "1" if first[1] else "0") != "0",
                   int(os.environ.get("DF3_DIFFUSION_CHUNK", str(first[2]))))]  # fmt: skip
    trainer = model_cfg = None
    for trunk_ckpt, diff_ckpt, chunk in ladder:
        os.environ["DF3_DIFFUSION_CKPT"] = "1" if diff_ckpt else "0"
        model_cfg = ModelConfig()
        model_cfg.msa_crop_size = N_MSA
        model_cfg.optim.use_gradient_checkpointing = trunk_ckpt
        if args.blocks:
            model_cfg.pairformer.num_layer = args.blocks
        train_cfg = TrainingConfig(**shared_train_settings(args.tokens), diffusion_chunk_size=chunk,
                                   per_rank_grad_clip=False, output_dir="/tmp/df3_bench")  # fmt: skip
        fits = 1
        try:
            trainer = Trainer(train_cfg, model_cfg, dist_info=info)

            def device_step(i, trainer=trainer):
                trainer.state.global_step = i
                loss, _, _ = trainer.micro_step(dict(dev_batch), num_recycles=recycles_for(i))
                trainer.engine.step_or_skip(trainer.state)

            def e2e_step(i, trainer=trainer):
                trainer.state.global_step = i
                trainer.train_step(dict(host_batch), num_recycles=recycles_for(i))

            for i in range(args.warmup):
                device_step(i)
            torch.cuda.synchronize()
        except torch.OutOfMemoryError:
            fits = 0
        if world > 1:
            import torch.distributed as dist

            flag = torch.tensor([fits], device=info.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            fits = int(flag.item())
        if fits:
            break
        trainer = None
        device_step = e2e_step = None
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    if trainer is None:
        raise SystemExit("out of memory under every memory policy")
    sampler = ClockSampler(info.local_rank)
    sampler.start()
    autograd_ops.launch_count(reset=True)
    sync = lambda: barrier(info)  # noqa: E731
    times = timed_loop(device_step, args.steps, args.warmup, sync, flush_buf)
    launches = autograd_ops.launch_count()
    clocks = sampler.stop()
    e2e_step(args.warmup - 1 if args.warmup else 0)  # pinned staging buffers allocated outside the timed region
    e2e_times = timed_loop(e2e_step, args.steps, args.warmup, sync, flush_buf)
    autograd_ops.check_status()  # a kernel wait that ran out anywhere in the run invalidates the numbers: fail loudly
    step_ms = reduce_max(sum(times) / len(times), world)
    e2e_ms = reduce_max(sum(e2e_times) / len(e2e_times), world)
    peak = torch.cuda.max_memory_allocated() / 2**30
    if info.is_main:
        emit(args, "ours", step_ms, e2e_ms, clocks, launches, batch_bytes(host_batch),
             {"activation_checkpointing": trunk_ckpt, "diffusion_checkpointing": diff_ckpt, "diffusion_chunk": chunk,
              "grad_transport": trainer.grad_sync.transport if world > 1 else "none",
              "optimizer_step": "one fused kernel" if trainer.grad_sync.fused_step_engine(trainer.optimizer) is not None else "classic",
              "trunk_graphs": _graph_state(trainer.model),
              "peak_mem_gib": round(peak, 1), "recycles": [recycles_for(args.warmup + i) for i in range(args.steps)]})  # fmt: skip
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def inference_features(args):
    """The synthetic job of an inference config in pinned host memory (unbatched, no ground truth)."""
    import torch

    from deepfold3_dev_b200.data.synthetic import synthetic_complex

    feats = synthetic_complex(args.cfg["chains"](args.tokens), num_msa=N_MSA, num_templates=N_TEMPLATES, seed=11, with_gt=False)
    return {k: (v.pin_memory() if isinstance(v, torch.Tensor) and torch.cuda.is_available() else v) for k, v in feats.items()}


def emit_inference(args, impl, step_ms, e2e_ms, clocks, launches, bytes_in, bytes_out, extra_cfg):
    c = args.cfg
    line = {
        "metric": c["metric"], "value": step_ms / 1e3, "unit": "s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": step_ms, "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random sequences, random-init weights)", "impl": impl,
        "config": {"model": "DeepFold3 default ModelConfig (48 Pairformer, 24 diffusion blocks, 368M params)", "seq_len": args.tokens,
                   "msa_rows": N_MSA, "templates": N_TEMPLATES, "recycles": c["recycles"], "sampler_steps": c["sampler_steps"],
                   "samples": c["samples"], "l2": "activations exceed L2; 256 MB buffer rewritten between predictions", **extra_cfg},
        "clocks": clocks,
        "e2e": {"value": e2e_ms / 1e3, "unit": "s", "h2d_bytes_per_step": bytes_in, "d2h_bytes_per_step": bytes_out,
                "ms_per_step": e2e_ms},
        "gpu_launches": launches,
    }  # fmt: skip
    print(json.dumps(line), flush=True)


def run_ours_inference(args):
    import torch

    sys.path.insert(0, ROOT)
    from deepfold3_dev_b200.config.schema import ModelConfig, OptimConfig
    from deepfold3_dev_b200.inference.runner import predict, predict_distributed
    from deepfold3_dev_b200.models.model import DeepFold3
    from deepfold3_dev_b200.ops import autograd_ops
    from deepfold3_dev_b200.parallel.dist import barrier, init_process_group

    info = init_process_group(timeout_s=1800.0)
    world = info.world_size
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    c = args.cfg
    if args.recycles >= 0:
        c["recycles"] = args.recycles
    if args.sampler_steps:
        c["sampler_steps"] = args.sampler_steps
    cfg = ModelConfig()
    cfg.optim = OptimConfig.inference()
    cfg.msa_crop_size = N_MSA
    cfg.diffusion.steps = c["sampler_steps"]
    cfg.diffusion.num_samples = c["samples"]
    if args.blocks:
        cfg.pairformer.num_layer = args.blocks
    torch.manual_seed(0)
    model = DeepFold3(cfg).to(info.device).eval()
    if world > 1:
        import torch.distributed as dist

        for t in list(model.parameters()) + list(model.buffers()):
            dist.broadcast(t.data, 0)
    host = inference_features(args)
    dev = {k: (v.to(info.device) if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
    flush_buf = torch.zeros(64 * 1024 * 1024, device=info.device)
    d2h = [0]

    def run(feats, seed, read: bool):
        if world > 1:
            _, out = predict_distributed(model, feats, seed, c["recycles"], c["samples"], info, use_bucket=False)
        else:
            out = predict(model, feats, seed, c["recycles"], c["samples"], info.device, use_bucket=False)
        if read and out is not None:  # the result of the prediction on the host: coordinates and every confidence head
            got = [t.to("cpu", non_blocking=True) for t in (out.atom_positions, out.plddt, out.pae, out.pde)]
            torch.cuda.synchronize()
            d2h[0] = sum(t.numel() * t.element_size() for t in got)

    device_step = lambda i: run(dev, i, False)  # noqa: E731
    e2e_step = lambda i: run(host, i, True)  # noqa: E731
    for i in range(args.warmup):
        device_step(i)
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    sampler = ClockSampler(info.local_rank)
    sampler.start()
    autograd_ops.launch_count(reset=True)
    sync = lambda: barrier(info)  # noqa: E731
    times = timed_loop(device_step, args.steps, args.warmup, sync, flush_buf)
    launches = autograd_ops.launch_count()
    clocks = sampler.stop()
    e2e_times = timed_loop(e2e_step, args.steps, args.warmup, sync, flush_buf)
    autograd_ops.check_status()
    step_ms = reduce_max(sum(times) / len(times), world)
    e2e_ms = reduce_max(sum(e2e_times) / len(e2e_times), world)
    bytes_out = int(reduce_max(float(d2h[0]), world))
    peak = torch.cuda.max_memory_allocated() / 2**30
    if info.is_main:
        comm = getattr(model.evoformer, "_axial_comm", None)
        emit_inference(args, "ours", step_ms, e2e_ms, clocks, launches, batch_bytes(host), bytes_out,
                       {"parallelism": f"trunk row-sharded over {world} GPUs ({comm.transport} exchange), samples dealt out" if world > 1 else "1 GPU",
                        "peak_mem_gib": round(peak, 1)})  # fmt: skip
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    infer = args.cfg["kind"] == "infer"
    if args.impl == "reference":
        from baseline import reference_arm

        (reference_arm.run_reference_inference if infer else reference_arm.run_reference)(args, sys.modules[__name__])
    elif infer:
        run_ours_inference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
