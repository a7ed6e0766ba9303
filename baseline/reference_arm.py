"""Reference arm of ``bench.py``: the unmodified reference package timed on the same config.

Only the reference's own code runs the model here: ``deepfold3.model.model.DeepFold3``,
``deepfold3.training.step.training_step``, ``wrap_ddp`` / ``build_optimizer`` / ``WrappedOptimizer``
/ ``EMA``. The package comes from ``baseline/_ref`` (a ``pip install --target`` of the reference
plus its ``src/deepfold3`` tree). Its data stack imports ``gemmi``, ``rdkit``,
``zstandard`` and ``pdbeccdutils`` at module import time; none is installable offline and none is
called on the synthetic-feature path, so inert stand-in modules are registered for the missing ones
before the import. The synthetic batch comes from this repository's generator (torch only).

Memory policy: the reference is given its fastest setting that fits the GPU. It is tried without activation
checkpointing and without diffusion chunking first (what this package's arm runs), then without checkpointing but
with its production diffusion chunk of 8, then with its production recipe (checkpointing + chunk 8); an attempt that
runs out of memory during warm-up is torn down and the next one is built. The JSON line says which one ran.
"""

from __future__ import annotations

import importlib
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF_PATH = os.path.join(HERE, "_ref")


class _Inert(types.ModuleType):
    """Stand-in for an uninstallable dependency: any attribute or call yields another stand-in."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        sub = _Inert(f"{self.__name__}.{name}")
        setattr(self, name, sub)
        sys.modules[sub.__name__] = sub
        return sub

    def __call__(self, *args, **kwargs):
        return _Inert(self.__name__ + "()")

    def __iter__(self):
        return iter(())

    def __mro_entries__(self, bases):
        return (object,)


def _stub_missing(names=("zstandard", "gemmi", "rdkit", "pdbeccdutils", "wandb")) -> list[str]:
    done = []
    for name in names:
        try:
            importlib.import_module(name)
        except Exception:  # noqa: BLE001
            mod = _Inert(name)
            mod.__path__ = []
            sys.modules[name] = mod
            done.append(name)
    return done


def unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def run_reference(args, bench) -> None:
    if not os.path.isdir(os.path.join(REF_PATH, "deepfold3", "model")):
        return unavailable("baseline/_ref does not hold the reference package (offline install missing)")
    sys.path.insert(0, REF_PATH)
    stubbed = _stub_missing()
    try:
        import torch
        import torch.distributed as dist
        from deepfold3.model.config import ModelConfig, TrainingConfig
        from deepfold3.model.model import DeepFold3
        from deepfold3.training.accumulator import AccumulationLoop
        from deepfold3.training.distributed import init_process_group
        from deepfold3.training.ema import EMA
        from deepfold3.training.optim import WrappedOptimizer, build_optimizer, wrap_ddp
        from deepfold3.training.scheduler import build_scheduler
        from deepfold3.training.state import TrainState, seed_everything
        from deepfold3.training.step import scaled_backward, training_step
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"reference import failed: {type(exc).__name__}: {exc}"[:300])
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")

    try:
        info = init_process_group(timeout_s=1800.0)
        world = info.world_size
        seed_everything(bench.SEED, info.rank)
        host_batch = bench.make_host_batch(info.rank, args.tokens, args.cfg["chains"])
        dev_batch = {k: v.to(info.device) for k, v in host_batch.items()}
        flush_buf = torch.zeros(64 * 1024 * 1024, device=info.device)
    except Exception as exc:  # noqa: BLE001 - set-up of the reference's own stack failed: report, do not crash
        if int(os.environ.get("RANK", "0")) == 0:
            unavailable(f"reference set-up failed: {type(exc).__name__}: {exc}"[:300])
        return
    opt_mode = os.environ.get("DF3_REF_OPTIM", "train")

    def build(checkpointing: bool, chunk: int):
        """The reference's model / DDP / optimizer / EMA stack under one memory policy, and a step function over it."""
        nonlocal opt_mode
        model_cfg = ModelConfig()
        model_cfg.msa_crop_size = bench.N_MSA
        if args.blocks:
            model_cfg.pairformer.num_layer = args.blocks
        o = model_cfg.optim
        o.use_gradient_checkpointing = checkpointing
        if opt_mode == "train":  # the kernel flags of the reference's production recipe (configs/initial.yaml:396-418)
            try:
                import triton  # noqa: F401

                o.use_fused_evo_attention = True
                o.use_fused_swiglu = True
                o.use_fused_triangle_mul = True
                o.use_fused_transition_pair = True
            except ImportError:
                opt_mode = "none (triton missing)"
        train_cfg = TrainingConfig(**bench.shared_train_settings(args.tokens), diffusion_chunk_size=chunk,
                                   per_rank_grad_clip=False)  # fmt: skip
        model = DeepFold3(model_cfg).to(info.device)
        model.train()
        ddp_model, _ = wrap_ddp(model, info, train_cfg)
        accumulator = AccumulationLoop(ddp_model=ddp_model, dist=info, num_steps=1, per_rank_clip=False)
        optimizer = build_optimizer(model, train_cfg)
        scheduler = build_scheduler(optimizer, train_cfg)
        ema = EMA(model, decay=train_cfg.ema_decay)
        scaler = torch.amp.GradScaler("cuda", enabled=False)
        wrapped = WrappedOptimizer(optimizer=optimizer, scheduler=scheduler, scaler=scaler, model=model, dist_info=info,
                                   cfg=train_cfg)  # fmt: skip
        state = TrainState()

        def one_step(i, features):
            state.global_step = i
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss, *_ = training_step(ddp_model, features, cfg=train_cfg, model_cfg=model_cfg, global_step=i,
                                         accumulator=accumulator, scaler=scaler, device=info.device)  # fmt: skip
            wrapped.add_microstep_loss(loss)
            with accumulator.step_context(is_sync_step=True):
                if loss.requires_grad:
                    scaled_backward(scaler, loss, 1)
            result = wrapped.step_or_skip(state)
            if result.advanced:
                ema.update(model)
            return loss

        return one_step

    ladder = [(False, 0), (False, 8), (True, 8)]
    if args.cfg.get("checkpointing"):  # crop 768: nothing fits without recomputation; try without diffusion chunking first
        ladder = [(True, 0), (True, 8)]
    if os.environ.get("DF3_REF_POLICY") == "production":
        ladder = [(True, 8)]
    one_step, policy = None, None
    for checkpointing, chunk in ladder:
        fits = 1
        try:
            one_step = build(checkpointing, chunk)
            for i in range(args.warmup):
                one_step(i, dict(dev_batch))
            torch.cuda.synchronize()
        except torch.OutOfMemoryError:
            fits = 0
        except Exception as exc:  # noqa: BLE001
            if info.rank == 0:
                unavailable(f"reference step failed ({opt_mode}, checkpointing={checkpointing}, chunk={chunk}): "
                            f"{type(exc).__name__}: {exc}"[:300])  # fmt: skip
            return
        if world > 1:  # every rank takes the same rung
            flag = torch.tensor([fits], device=info.device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            fits = int(flag.item())
        if fits:
            policy = (checkpointing, chunk)
            break
        one_step = None
        import gc

        gc.collect()
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    if policy is None:
        if info.rank == 0:
            unavailable("the reference ran out of memory under every memory policy, its production recipe included")
        return

    def device_step(i):
        one_step(i, dict(dev_batch))

    def e2e_step(i):
        loss = one_step(i, {k: v.to(info.device, non_blocking=True) for k, v in host_batch.items()})
        float(loss.item())

    def sync():
        if world > 1:
            dist.barrier()

    try:
        sampler = bench.ClockSampler(info.local_rank)
        sampler.start()
        times = bench.timed_loop(device_step, args.steps, args.warmup, sync, flush_buf)
        clocks = sampler.stop()
        e2e_times = bench.timed_loop(e2e_step, args.steps, args.warmup, sync, flush_buf)
    except Exception as exc:  # noqa: BLE001
        if info.rank == 0:
            unavailable(f"reference step failed ({opt_mode}): {type(exc).__name__}: {exc}"[:300])
        return
    step_ms = bench.reduce_max(sum(times) / len(times), world)
    e2e_ms = bench.reduce_max(sum(e2e_times) / len(e2e_times), world)
    peak = torch.cuda.max_memory_allocated() / 2**30
    if info.rank == 0:
        bench.emit(args, "reference", step_ms, e2e_ms, clocks, 0, bench.batch_bytes(host_batch),
                   {"reference_optim": opt_mode, "activation_checkpointing": policy[0], "diffusion_checkpointing": policy[0],
                    "diffusion_chunk": policy[1],
                    "stubbed_imports": stubbed, "peak_mem_gib": round(peak, 1),
                    "recycles": [bench.recycles_for(args.warmup + i) for i in range(args.steps)]})  # fmt: skip
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference_inference(args, bench) -> None:
    """The inference configs on the reference: its ``DeepFold3`` with its own ``OptimConfig.inference()`` preset (row
    chunking, tiled outer-product mean, its Triton kernels where importable). On several GPUs every process runs the whole
    trunk and its share of the samples, which is how the reference spreads work over GPUs (independent processes)."""
    if not os.path.isdir(os.path.join(REF_PATH, "deepfold3", "model")):
        return unavailable("baseline/_ref does not hold the reference package (offline install missing)")
    sys.path.insert(0, REF_PATH)
    stubbed = _stub_missing()
    try:
        import torch
        import torch.distributed as dist
        from deepfold3.model.config import ModelConfig, OptimConfig
        from deepfold3.model.model import DeepFold3
        from deepfold3.training.distributed import init_process_group
    except Exception as exc:  # noqa: BLE001
        return unavailable(f"reference import failed: {type(exc).__name__}: {exc}"[:300])
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    c = args.cfg
    if args.recycles >= 0:
        c["recycles"] = args.recycles
    if args.sampler_steps:
        c["sampler_steps"] = args.sampler_steps
    try:
        info = init_process_group(timeout_s=1800.0)
        world = info.world_size
        cfg = ModelConfig()
        cfg.optim = OptimConfig.inference()
        cfg.msa_crop_size = bench.N_MSA
        cfg.diffusion.steps = c["sampler_steps"]
        cfg.diffusion.num_samples = c["samples"]
        if args.blocks:
            cfg.pairformer.num_layer = args.blocks
        torch.manual_seed(0)
        model = DeepFold3(cfg).to(info.device).eval()
        host = bench.inference_features(args)
        dev = {k: (v.to(info.device) if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
        flush_buf = torch.zeros(64 * 1024 * 1024, device=info.device)
    except Exception as exc:  # noqa: BLE001
        if int(os.environ.get("RANK", "0")) == 0:
            unavailable(f"reference set-up failed: {type(exc).__name__}: {exc}"[:300])
        return
    share = len(range(info.rank, c["samples"], world))
    d2h = [0]

    def run(feats, seed, read):
        if share == 0:
            return
        feats = {k: (v.to(info.device, non_blocking=True) if isinstance(v, torch.Tensor) else v) for k, v in feats.items()}
        with torch.inference_mode(), torch.autocast("cuda", dtype=torch.bfloat16):
            out = model(feats, seed=seed * world + info.rank, num_recycles=c["recycles"], num_samples=share)
        if read:
            got = [t.to("cpu", non_blocking=True) for t in (out.atom_positions, out.plddt, out.pae, out.pde)]
            torch.cuda.synchronize()
            d2h[0] = sum(t.numel() * t.element_size() for t in got)

    def sync():
        if world > 1:
            dist.barrier()

    try:
        for i in range(args.warmup):
            run(dev, i, False)
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        sampler = bench.ClockSampler(info.local_rank)
        sampler.start()
        times = bench.timed_loop(lambda i: run(dev, i, False), args.steps, args.warmup, sync, flush_buf)
        clocks = sampler.stop()
        e2e_times = bench.timed_loop(lambda i: run(host, i, True), args.steps, args.warmup, sync, flush_buf)
    except torch.OutOfMemoryError:
        if info.rank == 0:
            unavailable("reference did not complete: out of memory on one B200 with its inference preset")
        return
    except Exception as exc:  # noqa: BLE001
        if info.rank == 0:
            unavailable(f"reference prediction failed: {type(exc).__name__}: {exc}"[:300])
        return
    step_ms = bench.reduce_max(sum(times) / len(times), world)
    e2e_ms = bench.reduce_max(sum(e2e_times) / len(e2e_times), world)
    bytes_out = int(bench.reduce_max(float(d2h[0]), world))
    peak = torch.cuda.max_memory_allocated() / 2**30
    if info.rank == 0:
        bench.emit_inference(args, "reference", step_ms, e2e_ms, clocks, 0, bench.batch_bytes(host), bytes_out,
                             {"parallelism": f"{world} independent processes, samples dealt out" if world > 1 else "1 GPU",
                              "reference_optim": "OptimConfig.inference()", "stubbed_imports": stubbed,
                              "peak_mem_gib": round(peak, 1)})  # fmt: skip
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
