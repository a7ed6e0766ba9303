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
    {"peer_reduce": peer_reduce, "peer_bench": peer_bench}[sys.argv[1]](info)
    dist.barrier()
    if info.rank == 0:
        print("WORKER_OK", sys.argv[1], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
