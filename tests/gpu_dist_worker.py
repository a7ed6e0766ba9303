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


def _pairformer_blocks(device, count, seed=5):
    from deepfold3_dev_b200.models.evoformer import PairFormerBlock
    from tests.helpers import wake_zero_init

    torch.manual_seed(seed)
    blocks = torch.nn.ModuleList(PairFormerBlock(128, 384) for _ in range(count)).eval()
    wake_zero_init(blocks)
    return blocks.to(device)


def axial_exchange(info):
    """Every re-layout on the peer-memory kernels equals its statement with NCCL collectives, bit for bit, over several
    calls (the receive heap is reused and grows)."""
    from deepfold3_dev_b200.parallel.axial import AxialComm

    peer, coll = AxialComm(info, "peer"), AxialComm(info, "collective")
    P, dev = info.world_size, info.device
    g = torch.Generator(device=dev).manual_seed(11 + info.rank)
    for n in (8, 32, 96):
        N = n * P
        z = torch.randn(2, n, N, 128, device=dev, generator=g).bfloat16()
        torch.testing.assert_close(peer.transpose(z), coll.transpose(z), atol=0, rtol=0)
        torch.testing.assert_close(peer.transpose(peer.transpose(z)), z, atol=0, rtol=0)
        planes = torch.randn(2, 16 * P, 2, n, N, device=dev, generator=g).bfloat16()
        mine = peer.rows_to_channels(planes)
        torch.testing.assert_close(mine, coll.rows_to_channels(planes), atol=0, rtol=0)
        back = peer.channels_to_rows(mine[0])
        torch.testing.assert_close(back, coll.channels_to_rows(mine[0]), atol=0, rtol=0)
        torch.testing.assert_close(back, planes[0], atol=0, rtol=0)
        bias = torch.randn(2, 4, n, N, device=dev, generator=g)
        torch.testing.assert_close(peer.all_gather(bias, 2), coll.all_gather(bias, 2), atol=0, rtol=0)
    peer.check()
    if info.rank == 0:
        print("AXIAL_EXCHANGE ok bootstrap=%s heap=%d MiB" % (peer.peer().bootstrap, peer.peer().heap_bytes >> 20), flush=True)


def axial_block(info):
    """Two Pairformer blocks at full width on row shards (bf16, own kernels, peer transport) against the same blocks
    unsharded on one GPU."""
    from deepfold3_dev_b200.parallel.axial import AxialComm, sharded_pairformer_stack

    dev, P = info.device, info.world_size
    blocks = _pairformer_blocks(dev, 2)
    B, N = 1, 256
    torch.manual_seed(3)
    pair, single = torch.randn(B, N, N, 128, device=dev), torch.randn(B, N, 384, device=dev)
    seq_mask = torch.ones(B, N, device=dev)
    seq_mask[0, -5:] = 0
    pair_mask = seq_mask[:, :, None] * seq_mask[:, None, :]
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        want_pair, want_single = pair.bfloat16(), single.bfloat16()
        for blk in blocks:
            want_pair, want_single = blk(want_pair, want_single, pair_mask, seq_mask)
        results = {}
        for transport in ("peer", "collective"):
            comm = AxialComm(info, transport)
            results[transport] = sharded_pairformer_stack(blocks, pair.bfloat16(), single.bfloat16(), pair_mask, seq_mask, comm)
            comm.check()
    for transport, (got_pair, got_single) in results.items():
        for got, want, what in ((got_pair, want_pair, "pair"), (got_single, want_single, "single")):
            err = (got.float() - want.float()).pow(2).mean().sqrt() / want.float().pow(2).mean().sqrt()
            assert float(err) < 1e-2, (transport, what, float(err))
    torch.testing.assert_close(results["peer"][0], results["collective"][0], atol=0, rtol=0)
    if info.rank == 0:
        print("AXIAL_BLOCK ok world=%d" % P, flush=True)


def axial_bench(info):
    """Device time per Pairformer block at a long token count: row-sharded over all ranks (peer kernels, NCCL) and, on
    rank 0 alone, unsharded. Token count from DF3_AXIAL_TOKENS (default 3072)."""
    from deepfold3_dev_b200.parallel.axial import AxialComm, sharded_pairformer_block

    dev, P = info.device, info.world_size
    N = int(os.environ.get("DF3_AXIAL_TOKENS", "3072"))
    blocks = _pairformer_blocks(dev, 2)
    torch.manual_seed(3)
    single = torch.randn(1, N, 384, device=dev).bfloat16()
    seq_mask = torch.ones(1, N, device=dev)
    pair_mask = torch.ones(1, N, N, device=dev)
    rows = torch.randn(1, N // P, N, 128, device=dev).bfloat16()
    out = {}
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        for transport in ("peer", "collective"):
            comm = AxialComm(info, transport)
            times = []
            for it in range(5):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                z, s = rows, single
                for blk in blocks:
                    z, s = sharded_pairformer_block(blk, z, s, pair_mask, seq_mask, comm)
                e1.record()
                e1.synchronize()
                if it >= 2:
                    times.append(e0.elapsed_time(e1) / len(blocks))
            comm.check()
            t = torch.tensor([sum(times) / len(times)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[transport] = float(t.item())
            del z, s
        torch.cuda.empty_cache()
        if info.rank == 0 and os.environ.get("DF3_AXIAL_SINGLE", "1") != "0":
            full = torch.randn(1, N, N, 128, device=dev).bfloat16()
            times = []
            for it in range(3):
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                z, s = full, single
                for blk in blocks:
                    z, s = blk(z, s, pair_mask, seq_mask)
                e1.record()
                e1.synchronize()
                if it >= 1:
                    times.append(e0.elapsed_time(e1) / len(blocks))
            out["one_gpu"] = sum(times) / len(times)
    if info.rank == 0:
        print("AXIAL_BENCH tokens=%d world=%d ms_per_block %s peak_gib=%.1f" % (
            N, P, " ".join(f"{k}={v:.2f}" for k, v in out.items()), torch.cuda.max_memory_allocated() / 2**30), flush=True)


def main():
    from deepfold3_dev_b200.parallel.dist import init_process_group

    info = init_process_group(timeout_s=120.0)
    {"peer_reduce": peer_reduce, "peer_bench": peer_bench, "fused_step": fused_step, "axial_exchange": axial_exchange,
     "axial_block": axial_block, "axial_bench": axial_bench}[sys.argv[1]](info)
    dist.barrier()
    if info.rank == 0:
        print("WORKER_OK", sys.argv[1], flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
