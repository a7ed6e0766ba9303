"""Multi-GPU worker for ``tests/test_gpu_multi.py`` (one process per GPU, launched with torch.distributed.run)."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peer_reduce(info):
    """The peer-memory reduction equals an NCCL all-reduce of the clipped gradients, several calls in a row."""
    from deepfold3_dev_b200.parallel.grad_sync import GradSync
    from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW

    torch.manual_seed(7)
    model = torch.nn.Sequential(torch.nn.Linear(300, 257), torch.nn.Linear(257, 1031), torch.nn.Linear(1031, 64)).to(info.device)
    opt = FlatAdamW(model, lr=1e-3, ema_decay=0.0)
    sync = GradSync(info, transport="peer")
    sync.attach(opt)
    for call in range(3):
        g = torch.Generator(device=info.device).manual_seed(100 * call + info.rank)
        local = torch.randn(opt.flat_grad.numel(), device=info.device, generator=g) * (1 + info.rank)
        opt.flat_grad.copy_(local)
        for per_rank in (False, True):
            opt.flat_grad.copy_(local)
            ref = local.clone()
            if per_rank:
                n = ref.double().norm().float()
                ref.mul_(torch.clamp(0.5 / (n + 1e-6), max=1.0))
            dist.all_reduce(ref, op=dist.ReduceOp.AVG)
            local_norm, global_norm, scale = sync.clip_and_average(opt, 0.5, per_rank)
            torch.testing.assert_close(opt.flat_grad, ref, rtol=1e-5, atol=1e-6)
            got = global_norm if per_rank else local_norm
            torch.testing.assert_close(got, ref.double().norm().float(), rtol=1e-4, atol=1e-6)
    sync._peer.check()
    # every .grad view sits in the symmetric buffer
    base = opt.flat_grad.data_ptr()
    assert all(p.grad.data_ptr() == base + 4 * o for p, o in zip(opt.params, opt.offsets))


def fused_step(info):
    """The one-kernel optimizer step on every rank equals NCCL all-reduce(AVG) + clip + torch AdamW + EMA lerp, in both
    clipping modes, and skips on every rank when one rank flags a non-finite loss."""
    from deepfold3_dev_b200.config.schema import TrainingConfig
    from deepfold3_dev_b200.parallel.grad_sync import GradSync
    from deepfold3_dev_b200.training.engine import OptimizerEngine
    from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW
    from deepfold3_dev_b200.training.scheduler import build_scheduler
    from deepfold3_dev_b200.training.state import TrainState

    def build():
        torch.manual_seed(7)
        return torch.nn.Sequential(torch.nn.Linear(300, 257), torch.nn.Linear(257, 1031), torch.nn.Linear(1031, 64)).to(info.device)

    for per_rank in (False, True):
        cfg = TrainingConfig(lr=1e-2, warmup_steps=0, grad_clip_norm=0.5, per_rank_grad_clip=per_rank, ema_decay=0.9,
                             max_consecutive_nan_skips=0)  # fmt: skip
        model, ref_model = build(), build()
        opt = FlatAdamW(model, lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, ema_decay=cfg.ema_decay)
        sync = GradSync(info, transport="peer")
        sync.attach(opt)
        engine = OptimizerEngine(opt, build_scheduler(opt, cfg), info, cfg, grad_sync=sync)
        assert sync.fused_step_engine(opt) is not None
        ref = torch.optim.AdamW(ref_model.parameters(), lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, weight_decay=0.0)
        shadow = [p.detach().clone() for p in ref_model.parameters()]
        state = TrainState()
        for step in range(4):
            g = torch.Generator(device=info.device).manual_seed(100 * step + info.rank)
            x = torch.randn(32, 300, device=info.device, generator=g) * (1 + info.rank)
            model(x).pow(2).sum().backward()
            ref_model(x).pow(2).sum().backward()
            bad_loss = step == 2 and info.rank == info.world_size - 1
            engine.add_microstep_loss(torch.tensor(float("nan") if bad_loss else 1.0, device=info.device))
            # reference: what the classic sequence does with NCCL
            grads = [p.grad for p in ref_model.parameters()]
            flat = torch.cat([t.reshape(-1) for t in grads])
            if per_rank:
                n = flat.double().norm().float()
                flat.mul_(torch.clamp(0.5 / (n + 1e-6), max=1.0))
            dist.all_reduce(flat, op=dist.ReduceOp.AVG)
            if not per_rank:
                n = flat.double().norm().float()
                flat.mul_(torch.clamp(0.5 / (n + 1e-6), max=1.0))
            o = 0
            for t in grads:
                t.copy_(flat[o : o + t.numel()].view_as(t))
                o += t.numel()
            engine.step_or_skip(state)
            res = engine.resolve(state)
            if step == 2:
                assert res is not None and not res.advanced and res.reason == "loss" and res.nan_ranks == [info.world_size - 1], res
            else:
                assert res is not None and res.advanced, res
                ref.step()
                torch._foreach_lerp_(shadow, [p.detach() for p in ref_model.parameters()], 1 - cfg.ema_decay)
            ref.zero_grad()
        assert state.effective_step == 3 and opt.step_count == 3
        for p, q in zip(model.parameters(), ref_model.parameters()):
            torch.testing.assert_close(p, q, atol=2e-6, rtol=1e-4)
        ema = opt.ema_state_dict()["shadow"]
        for (name, _), sh in zip(model.named_parameters(), shadow):
            torch.testing.assert_close(ema[name], sh, atol=2e-6, rtol=1e-4)
        sync._peer.check()
        if info.rank == 0:
            print("FUSED_STEP ok per_rank_clip=%s bootstrap=%s" % (per_rank, sync._peer.bootstrap), flush=True)


def peer_bench(info):
    """Device time of the peer-memory reduction against NCCL all-reduce + norm on a 368 M element buffer."""
    from deepfold3_dev_b200.parallel.grad_sync import GradSync
    from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW

    n = 368 * 1024 * 1024
    model = torch.nn.Linear(1024, n // 1024, bias=False).to(info.device)
    opt = FlatAdamW(model, lr=1e-3, ema_decay=0.0)
    opt.flat_grad.normal_()
    results = {}
    for transport in ("collective", "peer"):
        sync = GradSync(info, transport=transport)
        sync.attach(opt)
        times = []
        for it in range(8):
            opt.flat_grad.normal_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            sync.clip_and_average(opt, 10.0, False)
            e1.record()
            e1.synchronize()
            if it >= 3:
                times.append(e0.elapsed_time(e1))
        t = torch.tensor([sum(times) / len(times)], device=info.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[transport] = float(t.item())
    if info.rank == 0:
        gb = 4 * n / 1e9
        w = info.world_size
        for k, ms in results.items():
            print(f"PEER_BENCH world={w} {k}: {ms:.3f} ms  bus bandwidth {2 * (w - 1) / w * gb / ms * 1e3:.0f} GB/s", flush=True)


def main():
    from deepfold3_dev_b200.parallel.dist import init_process_group

    info = init_process_group(timeout_s=120.0)
    {"peer_reduce": peer_reduce, "peer_bench": peer_bench, "fused_step": fused_step}[sys.argv[1]](info)
    dist.barrier()
    if info.rank == 0:
        print("WORKER_OK", sys.argv[1], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
