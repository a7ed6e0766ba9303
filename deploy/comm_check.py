"""Collective bandwidth check for a freshly allocated set of nodes.

Run it before a long training job, with the same launcher and environment as the job itself:

    python -m torch.distributed.run --nproc-per-node 8 [--nnodes N ...] deploy/comm_check.py
    python -m torch.distributed.run --nproc-per-node 8 deploy/comm_check.py --sizes-mib 1 64 1024 --peer

It times all-reduce, all-gather, reduce-scatter and all-to-all through ``torch.distributed`` (NCCL on GPUs, gloo on
CPU) for a few message sizes, on the device with CUDA events, and prints the algorithm bandwidth and the bus
bandwidth (the figure that is comparable across rank counts) as the maximum time over ranks. ``--peer`` adds the
package's own peer-memory gradient reduction and axial exchange kernels (one node only). ``--min-busbw`` turns the
run into a gate: the exit code is 1 when the 1-GPU-per-rank all-reduce at the largest size stays under that many GB/s,
which is how a batch script refuses to start a long run on a fabric that fell back to TCP.

The reference answers the same question with the `nccl-tests` binary under mpirun (kakao/nccl-tests.yaml) and with an
all-reduce inside its Slurm pre-flight (hangang/check.sbatch); this script needs nothing but the training image.
"""

from __future__ import annotations

import argparse
import json
import os
import socket
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _timed(fn, device: torch.device, iters: int, warmup: int) -> float:
    """Seconds per call: device time on CUDA, wall time on CPU; maximum over ranks."""
    for _ in range(warmup):
        fn()
    if device.type == "cuda":
        torch.cuda.synchronize(device)
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(iters):
            fn()
        stop.record()
        torch.cuda.synchronize(device)
        seconds = start.elapsed_time(stop) / 1e3 / iters
    else:
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        seconds = (time.perf_counter() - t0) / iters
    worst = torch.tensor([seconds], dtype=torch.float64, device=device if device.type == "cuda" else "cpu")
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return float(worst.item())


def bus_factor(op: str, world: int) -> float:
    """Bus bandwidth = algorithm bandwidth x this factor (the convention of nccl-tests)."""
    if op == "all_reduce":
        return 2.0 * (world - 1) / world
    return (world - 1) / world  # all_gather, reduce_scatter, all_to_all


def sweep(device: torch.device, sizes_mib, iters: int, warmup: int, dtype=torch.bfloat16):
    world = dist.get_world_size()
    rows = []
    for mib in sizes_mib:
        n = int(mib * 2**20) // dtype.itemsize if dtype.is_floating_point else int(mib * 2**20)
        n = max(world, n // world * world)
        full = torch.ones(n, dtype=dtype, device=device)
        part = torch.ones(n // world, dtype=dtype, device=device)
        other = torch.empty_like(full)
        ops = {
            "all_reduce": lambda: dist.all_reduce(full),
            "all_gather": lambda: dist.all_gather_into_tensor(other, part),
            "reduce_scatter": lambda: dist.reduce_scatter_tensor(part, full),
            "all_to_all": lambda: dist.all_to_all_single(other, full),
        }
        if dist.get_backend() == "gloo":
            # gloo has no reduce-scatter and reduces bf16 slowly; keep the two it does well
            full, other, part = full.float(), other.float(), part.float()
            ops = {"all_reduce": lambda: dist.all_reduce(full),
                   "all_gather": lambda: dist.all_gather_into_tensor(other, part)}  # fmt: skip
        for name, fn in ops.items():
            seconds = _timed(fn, device, iters, warmup)
            nbytes = full.numel() * full.element_size()
            alg = nbytes / seconds / 1e9
            rows.append({"op": name, "mib": nbytes / 2**20, "us": seconds * 1e6, "algbw_gbs": alg, "busbw_gbs": alg * bus_factor(name, world)})
            full.fill_(1)  # repeated in-place sums would overflow bf16
    return rows


def peer_rows(device: torch.device, sizes_mib, iters: int, warmup: int, transport: str = "peer"):
    """The package's own one-node transports: gradient reduction and the rows<->channels exchange."""
    from deepfold3_dev_b200.parallel.axial import AxialComm
    from deepfold3_dev_b200.parallel.dist import DistInfo, on_one_node

    world, rank = dist.get_world_size(), dist.get_rank()
    info = DistInfo(rank, device.index or 0, world, device, dist.get_backend())
    if not on_one_node(info):
        return [{"op": "peer", "skipped": "ranks span several hosts"}]
    comm = AxialComm(info, transport)
    rows = []
    for mib in sizes_mib:
        channels = 128
        n = int((mib * 2**20 / 2 / channels) ** 0.5) // world * world
        if n < world:
            continue
        x = torch.randn(1, n // world, n, channels, device=device, dtype=torch.bfloat16)         # row shard [B, n, N, C]
        planes = torch.randn(1, channels, 1, n // world, n, device=device, dtype=torch.bfloat16)  # channel planes [G, C, B, n, N]
        for name, fn in {"peer_all_gather": lambda: comm.all_gather(x, 1), "peer_transpose": lambda: comm.transpose(x),
                         "peer_rows_to_channels": lambda: comm.rows_to_channels(planes)}.items():  # fmt: skip
            seconds = _timed(fn, device, iters, warmup)
            nbytes = x.numel() * x.element_size() * (world if name == "peer_all_gather" else 1)
            alg = nbytes / seconds / 1e9
            rows.append({"op": name, "mib": nbytes / 2**20, "us": seconds * 1e6, "algbw_gbs": alg,
                         "busbw_gbs": alg * (world - 1) / world})  # fmt: skip
    comm.check()
    return rows


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=[1, 16, 256, 1024])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--peer", action="store_true", help="also time the package's peer-memory kernels (one node)")
    ap.add_argument("--peer-transport", choices=["peer", "collective"], default="peer",
                    help="exchange transport for --peer: the peer-memory kernels, or their collective statement (also runs on CPU)")
    ap.add_argument("--min-busbw", type=float, default=0.0, help="fail when the largest all-reduce is below this many GB/s")
    ap.add_argument("--json", type=str, default=None, help="write the table here (rank 0)")
    args = ap.parse_args(argv)

    use_cuda = torch.cuda.is_available()
    local = int(os.environ.get("LOCAL_RANK", 0))
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group("nccl" if use_cuda else "gloo", **({"device_id": device} if use_cuda else {}))
    rank, world = dist.get_rank(), dist.get_world_size()

    hosts: list = [None] * world
    dist.all_gather_object(hosts, (socket.gethostname(), torch.cuda.get_device_name(device) if use_cuda else "cpu"))
    rows = sweep(device, args.sizes_mib, args.iters, args.warmup)
    if args.peer and (use_cuda or args.peer_transport == "collective"):
        rows += peer_rows(device, args.sizes_mib, args.iters, args.warmup, args.peer_transport)

    status = 0
    if rank == 0:
        nodes = sorted({h for h, _ in hosts})
        print(f"ranks {world} on {len(nodes)} host(s): {', '.join(nodes)}; device {hosts[0][1]}; backend {dist.get_backend()}")
        print(f"{'op':24s}{'MiB':>10s}{'us':>12s}{'algbw GB/s':>14s}{'busbw GB/s':>14s}")
        for r in rows:
            if "skipped" in r:
                print(f"{r['op']:24s} skipped: {r['skipped']}")
                continue
            print(f"{r['op']:24s}{r['mib']:10.1f}{r['us']:12.1f}{r['algbw_gbs']:14.1f}{r['busbw_gbs']:14.1f}")
        big = [r for r in rows if r.get("op") == "all_reduce"]
        if args.min_busbw and big and big[-1]["busbw_gbs"] < args.min_busbw:
            print(f"FAIL: all-reduce bus bandwidth {big[-1]['busbw_gbs']:.1f} GB/s < {args.min_busbw} GB/s")
            status = 1
        if args.json:
            with open(args.json, "w") as fh:
                json.dump({"world": world, "hosts": nodes, "rows": rows}, fh, indent=1)
    flag = torch.tensor([status], device=device if use_cuda else "cpu")
    dist.broadcast(flag, 0)
    dist.destroy_process_group()
    return int(flag.item())


if __name__ == "__main__":
    raise SystemExit(main())
