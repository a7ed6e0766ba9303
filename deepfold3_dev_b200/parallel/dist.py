"""Process-group bootstrap and the small host-side collectives of the training loop.

One process per GPU, rendezvous from ``RANK / WORLD_SIZE / LOCAL_RANK /
MASTER_*`` (reference: training/distributed.py:26-97). The backend is ``nccl``
on GPUs and ``gloo`` on CPU, so every multi-process path is testable without a
GPU. Control-plane collectives (NaN consensus, shutdown flag, meters) stay on
``torch.distributed``; the gradient path has its own engine in
``parallel/grad_sync.py``.
"""

from __future__ import annotations

import datetime
import logging
import os
import platform
import signal
from contextlib import contextmanager
from dataclasses import dataclass

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


@dataclass
class DistInfo:
    rank: int = 0
    local_rank: int = 0
    world_size: int = 1
    device: torch.device = torch.device("cpu")
    backend: str | None = None

    @property
    def is_distributed(self) -> bool:
        return self.world_size > 1

    @property
    def is_main(self) -> bool:
        return self.rank == 0


def init_process_group(timeout_s: float = 600.0, device: str | None = None) -> DistInfo:
    """Join the job described by the environment; single-process when ``WORLD_SIZE`` is absent or 1."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    use_cuda = torch.cuda.is_available() and device != "cpu"
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
    else:
        dev = torch.device("cpu")
    if world <= 1:
        return DistInfo(rank, local, 1, dev, None)
    backend = "nccl" if use_cuda else "gloo"
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = dict(backend=backend, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        if use_cuda:
            kwargs["device_id"] = dev
        dist.init_process_group(**kwargs)
    return DistInfo(rank, local, world, dev, backend)


_ONE_NODE: dict[int, bool] = {}


def on_one_node(info: DistInfo) -> bool:
    """True when every rank of the job runs on the same host (a collective call on first use; cached afterwards).

    CUDA-IPC peer mappings exist only between the GPUs of one host, so the peer-memory transports are the default only
    when this holds; a job that spans hosts reduces gradients through NCCL instead.
    """
    if not info.is_distributed:
        return True
    if info.world_size not in _ONE_NODE:
        import socket

        names: list = [None] * info.world_size
        dist.all_gather_object(names, socket.gethostname())
        _ONE_NODE[info.world_size] = len(set(names)) == 1
    return _ONE_NODE[info.world_size]


def destroy_process_group_safely(info: DistInfo) -> None:
    if info.is_distributed and dist.is_initialized():
        try:
            barrier(info)
        finally:
            dist.destroy_process_group()


def barrier(info: DistInfo) -> None:
    if not info.is_distributed:
        return
    if info.backend == "nccl":
        dist.barrier(device_ids=[info.local_rank])
    else:
        dist.barrier()


@contextmanager
def collective_guard(name: str, info: DistInfo):
    """Named entry and exit barriers around a region every rank must pass together.

    A desynchronised rank then fails within the process-group timeout with the
    region's name in the error, instead of hanging in an anonymous collective
    (reference: training/collective_guard.py:33-61).
    """
    if not info.is_distributed:
        yield
        return
    for side in ("entry", "exit"):
        try:
            barrier(info)
        except RuntimeError as exc:
            raise RuntimeError(f"collective_guard({name!r}) {side} barrier: {exc}") from exc
        if side == "entry":
            yield


def all_gather_scalar(value: torch.Tensor, info: DistInfo) -> torch.Tensor:
    """``[world_size]`` tensor holding every rank's 1-element ``value``."""
    v = value.reshape(1)
    if not info.is_distributed:
        return v
    out = torch.zeros(info.world_size, device=v.device, dtype=v.dtype)
    dist.all_gather_into_tensor(out, v)
    return out


class ShutdownCoordinator:
    """SIGTERM / SIGINT / stop-file → a flag every rank agrees on each micro-step (reference: signals.py:32-72)."""

    def __init__(self, info: DistInfo, install_handlers: bool = True) -> None:
        self.dist = info
        self.requested = False
        self._stop_file = os.environ.get("DF3_STOP_FILE")
        self._flag = torch.zeros(1, dtype=torch.int32, device=info.device)
        if install_handlers and platform.system() != "Windows":
            try:
                signal.signal(signal.SIGTERM, lambda *_: self._set())
                signal.signal(signal.SIGINT, lambda *_: self._set())
            except ValueError:  # not the main thread
                pass

    def _set(self) -> None:
        self.requested = True

    def tick(self) -> bool:
        if self._stop_file and self.dist.is_main and not self.requested and os.path.exists(self._stop_file):
            logger.info("Stop file %s found, shutting down", self._stop_file)
            self.requested = True
        if self.dist.is_distributed:
            self._flag.fill_(int(self.requested))
            dist.all_reduce(self._flag, op=dist.ReduceOp.MAX)
            self.requested = bool(self._flag.item())
        return self.requested


class CheckpointRequestHandler:
    """SIGUSR2 = "write a checkpoint at the next boundary" (rank-0 flag, polled and cleared by the loop)."""

    def __init__(self) -> None:
        self._requested = False
        if platform.system() != "Windows":
            try:
                signal.signal(signal.SIGUSR2, lambda *_: self._set())
            except ValueError:
                pass

    def _set(self) -> None:
        self._requested = True

    def consume(self) -> bool:
        out, self._requested = self._requested, False
        return out
