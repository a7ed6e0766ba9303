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


def main():
    from deepfold3_dev_b200.parallel.dist import init_process_group

    info = init_process_group(timeout_s=120.0)
    {"peer_reduce": peer_reduce}[sys.argv[1]](info)
    dist.barrier()
    if info.rank == 0:
        print("WORKER_OK", sys.argv[1], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
