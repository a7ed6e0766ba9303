"""All-to-all and all-gather of sharded activations over NVLink peer memory (``ops/csrc/peer_exchange.cu``).

Each re-layout the axial-sharded Pairformer needs is one strided push pattern: three loop levels with source and
destination strides, a contiguous inner run, a source offset per destination rank and a destination offset fixed by
the sender. ``plan_*`` build those patterns (pure integer arithmetic, checked on the CPU by ``emulate``); ``PeerExchange``
owns the receive heap and control block, shares them with the other ranks once (CUDA IPC handles, symmetric memory as
the fallback) and launches the kernels. The reference has no counterpart: it never shards one sample.
"""

from __future__ import annotations

import dataclasses
import logging
import math

import torch
import torch.distributed as dist

from .dist import DistInfo
from .peer_reduce import CTRL_BYTES, MAX_WORLD, _share_over_ipc, _share_over_symmetric_memory

logger = logging.getLogger(__name__)


@dataclasses.dataclass(frozen=True)
class Plan:
    """Element ``(i0, i1, i2, v)`` of the contribution for rank ``q`` is read at ``q * src_q + sum(i * sstr) + v`` and
    lands at ``dst_base + sum(i * dstr) + v`` of rank ``q``'s result (all in elements)."""

    out_shape: tuple
    counts: tuple
    sstr: tuple
    dstr: tuple
    inner: int
    src_q: int
    dst_base: int


def plan_all_gather(shape, dim: int, rank: int, world: int) -> Plan:
    dim = dim % len(shape)
    pre, m, post = math.prod(shape[:dim]), shape[dim], math.prod(shape[dim + 1 :])
    out = (*shape[:dim], world * m, *shape[dim + 1 :])
    return Plan(out, (1, 1, pre), (0, 0, m * post), (0, 0, world * m * post), m * post, 0, rank * m * post)


def plan_transpose(shape, rank: int, world: int) -> Plan:
    """Row shard ``[B, n, N, C]`` of ``z`` -> row shard of ``z^T`` (``out[b, j, i] = z[b, i, rank * n + j]``)."""
    B, n, N, C = shape
    if N != n * world:
        raise ValueError(f"row shard {tuple(shape)} does not match {world} ranks")
    return Plan((B, n, N, C), (B, n, n), (n * N * C, N * C, C), (n * N * C, C, N * C), C, n * C, rank * n * C)


def plan_rows_to_channels(shape, rank: int, world: int) -> Plan:
    """Channel planes of this rank's rows ``[G, C, B, n, N]`` -> all rows of this rank's channels ``[G, C / P, B, N, N]``."""
    G, C, B, n, N = shape
    if C % world or N != n * world:
        raise ValueError(f"planes {tuple(shape)} cannot be split over {world} ranks")
    cp = C // world
    return Plan((G, cp, B, N, N), (G, cp, B), (C * B * n * N, B * n * N, n * N), (cp * B * N * N, B * N * N, N * N), n * N,
                cp * B * n * N, rank * n * N)  # fmt: skip


def plan_channels_to_rows(shape, rank: int, world: int) -> Plan:
    """All rows of this rank's channels ``[C / P, B, N, N]`` -> every channel of this rank's rows ``[C, B, n, N]``."""
    cp, B, N, N2 = shape
    if N % world or N != N2:
        raise ValueError(f"planes {tuple(shape)} cannot be split over {world} ranks")
    n = N // world
    return Plan((cp * world, B, n, N), (1, cp, B), (0, B * N * N, N * N), (0, B * n * N, n * N), n * N, n * N, rank * cp * B * n * N)


def emulate(plans: list[Plan], sources: list[torch.Tensor]) -> list[torch.Tensor]:
    """What the push kernel does, on the host and for all ranks at once: ``sources[p]`` pushed with ``plans[p]``. Returns
    every rank's result. Used to check the patterns against the collective statement of the same re-layout."""
    world = len(plans)
    outs = [torch.empty(math.prod(plans[q].out_shape), dtype=sources[0].dtype) for q in range(world)]
    for p, (plan, src) in enumerate(zip(plans, sources)):
        flat = src.contiguous().view(-1)
        n0, n1, n2 = plan.counts
        i0, i1, i2, v = torch.meshgrid(torch.arange(n0), torch.arange(n1), torch.arange(n2), torch.arange(plan.inner), indexing="ij")
        s_off = i0 * plan.sstr[0] + i1 * plan.sstr[1] + i2 * plan.sstr[2] + v
        d_off = plan.dst_base + i0 * plan.dstr[0] + i1 * plan.dstr[1] + i2 * plan.dstr[2] + v
        for q in range(world):
            outs[q][d_off.reshape(-1)] = flat[(q * plan.src_q + s_off).reshape(-1)]
    return [o.view(plans[q].out_shape) for q, o in enumerate(outs)]


class PeerExchange:
    def __init__(self, info: DistInfo, heap_bytes: int = 64 << 20):
        from ..ops import native

        if not native.require().has("peer_exchange"):
            raise RuntimeError("the extension was built without the peer exchange kernels")
        if not 2 <= info.world_size <= MAX_WORLD:
            raise ValueError(f"peer exchange runs on 2 to {MAX_WORLD} ranks of one node")
        self.info = info
        self._keep = []  # every heap ever shared stays mapped on the peers: keep them alive
        self.heap_bytes = 0
        self.bootstrap = None
        self.status = torch.zeros(1, dtype=torch.int32, device=info.device)
        self.scratch = torch.zeros(4, dtype=torch.int32, device=info.device)
        self.seq = 0
        self.ctrl_ptrs = self._share(CTRL_BYTES)[1]
        self._grow(heap_bytes)

    def _share(self, nbytes: int):
        info = self.info
        buf = ptrs = None
        try:
            buf, ptrs = _share_over_ipc(info, nbytes)
            how = "cuda-ipc"
        except Exception as exc:  # noqa: BLE001 - the choice has to be the same on every rank
            logger.warning("CUDA IPC sharing of the exchange heap failed (%r)", exc)
        ok = torch.tensor([1 if buf is not None else 0], device=info.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0:
            buf, ptrs, handle = _share_over_symmetric_memory(info, nbytes)
            self._keep.append(handle)
            how = "symmetric-memory"
        buf.zero_()
        self._keep.append(buf)
        self.bootstrap = how
        torch.cuda.synchronize(info.device)
        dist.barrier()
        return buf, ptrs

    def _grow(self, nbytes: int) -> None:
        """A larger heap on every rank (all ranks run the same sequence of exchanges, so they grow together)."""
        nbytes = max(int(nbytes), 2 * self.heap_bytes)
        nbytes = (nbytes + (1 << 21) - 1) >> 21 << 21
        _, self.heap_ptrs = self._share(nbytes)
        self.heap_bytes = nbytes

    def run(self, src: torch.Tensor, plan: Plan, spin_limit: int = 0) -> torch.Tensor:
        src = src.contiguous()
        out = src.new_empty(plan.out_shape)
        nbytes = out.numel() * out.element_size()
        if nbytes > self.heap_bytes:
            self._grow(nbytes)
        self.seq += 1
        torch.ops.df3.peer_exchange(src, out, self.heap_ptrs, self.ctrl_ptrs, self.heap_bytes, self.scratch, self.status,
                                    self.info.rank, self.info.world_size, self.seq, list(plan.counts), list(plan.sstr),
                                    list(plan.dstr), plan.inner, plan.src_q, plan.dst_base, int(spin_limit))  # fmt: skip
        return out

    def all_gather(self, x, dim):
        return self.run(x, plan_all_gather(tuple(x.shape), dim, self.info.rank, self.info.world_size))

    def transpose(self, x):
        return self.run(x, plan_transpose(tuple(x.shape), self.info.rank, self.info.world_size))

    def rows_to_channels(self, x):
        return self.run(x, plan_rows_to_channels(tuple(x.shape), self.info.rank, self.info.world_size))

    def channels_to_rows(self, x):
        return self.run(x, plan_channels_to_rows(tuple(x.shape), self.info.rank, self.info.world_size))

    def check(self) -> None:
        """Raise if a flag wait ran out since the last check (reads the status word: synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer exchange: a wait for another rank's flag timed out (status {code}); results are undefined")
