"""Data-parallel gradient reduction over the flat gradient buffer.

The reference reduces gradients either through DDP's 25 MB buckets or, in
per-rank-clip mode, with one coalesced ``all_reduce(AVG)`` after a flatten /
unflatten round trip (training/optim.py:69-108, :405-412). Here gradients
already live in one flat fp32 buffer (``FlatAdamW.flat_grad``), so a reduction
is one collective with no packing. Two transports:

* ``collective``: ``torch.distributed.all_reduce`` (NCCL on GPUs, gloo on CPU).
  Always available; the correctness oracle for the other and the default on CPU.
* ``peer``: the sm_100a kernel in ``ops/csrc/peer_reduce.cu`` working on
  NVLink peer mappings of every rank's buffer: each rank sums its slice of all
  ranks' gradients (applying each source rank's clip coefficient), writes the
  averaged slice back to every rank and accumulates the squared norm, in one
  launch. The default for NCCL process groups; ``DF3_COMM=collective`` switches it off.

Both give every rank the same averaged gradient and its global norm.
"""

from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .dist import DistInfo, on_one_node


class GradSync:
    def __init__(self, info: DistInfo, transport: str | None = None):
        self.info = info
        # NCCL ranks on one node default to the peer-memory kernel; everything else (CPU, several hosts) to the collective
        default = "collective"
        if info.is_distributed and info.backend == "nccl" and transport is None and "DF3_COMM" not in os.environ:
            default = "peer" if on_one_node(info) else "collective"
        self.explicit = transport is not None or "DF3_COMM" in os.environ
        self.transport = transport or os.environ.get("DF3_COMM", default)
        self._peer = None

    def _peer_engine(self, opt):
        if self._peer is None:
            from .peer_reduce import PeerReducer

            self._peer = PeerReducer(self.info, opt)
        return self._peer

    def attach(self, opt) -> None:
        """Peer transport: move the optimizer's gradient buffer into peer-mapped memory now (a collective call).

        When the transport was asked for explicitly (``DF3_COMM=peer`` or the ``transport`` argument) a failure to set it
        up is an error; only the implicit default falls back to the collective, and says so.
        """
        if self.transport == "peer" and self.info.is_distributed and opt.flat_grad.is_cuda:
            try:
                self._peer_engine(opt)
            except Exception as exc:  # noqa: BLE001
                if self.explicit:
                    raise RuntimeError(f"DF3_COMM=peer: the peer-memory gradient transport could not be set up: {exc!r}") from exc
                import logging

                logging.getLogger(__name__).warning("peer-memory gradient transport unavailable (%r); using NCCL", exc)
                self.transport, self._peer = "collective", None

    def fused_step_engine(self, opt):
        """The peer engine when the whole optimizer step can run as its one fused kernel, else ``None``: CUDA buffers,
        plain ``FlatAdamW`` (the schedule-free update has its own sequence), the peer transport (or a single process),
        and not switched off with ``DF3_FUSED_STEP=0``."""
        from ..training.flat_optimizer import FlatAdamW

        if type(opt) is not FlatAdamW or not opt.flat_grad.is_cuda or os.environ.get("DF3_FUSED_STEP", "1") == "0":
            return None
        if self.info.is_distributed and self.transport != "peer":
            return None
        try:
            return self._peer_engine(opt)
        except Exception:  # noqa: BLE001 - single process without the extension: the classic sequence still works
            if self.info.is_distributed:
                raise
            return None

    @torch.no_grad()
    def clip_and_average(self, opt, clip_norm: float, per_rank_clip: bool, fp64_norm: bool = True):
        """Average ``opt.flat_grad`` over ranks and derive the factor the optimizer multiplies gradients by.

        Returns ``(local_norm, global_norm_or_None, grad_scale)``:

        * classic mode: gradients are averaged first, ``local_norm`` is the norm of the average and
          ``grad_scale = min(1, clip / (norm + 1e-6))`` is applied inside the optimizer kernel;
        * per-rank mode: every rank scales its own gradient by its own clip coefficient before the
          average; ``local_norm`` is this rank's pre-clip norm, ``global_norm`` the norm of the average,
          and ``grad_scale`` is 1.

        Non-finite norms give ``grad_scale = 1`` and leave the skip decision to the caller.
        """
        info = self.info
        clip = clip_norm if clip_norm and clip_norm > 0 else float("inf")

        def coef(norm):
            c = torch.clamp(clip / (norm + 1e-6), max=1.0)
            return torch.where(torch.isfinite(norm), c, torch.ones_like(c))

        if not info.is_distributed:
            norm = opt.grad_norm(fp64_norm)
            return norm, None, coef(norm)
        if per_rank_clip:
            local = opt.grad_norm(fp64_norm)
            if self.transport == "peer" and opt.flat_grad.is_cuda:
                global_norm = self._peer_engine(opt).all_reduce_mean(opt.flat_grad, coef(local))
            else:
                opt.flat_grad.mul_(coef(local))
                self._all_reduce_mean(opt.flat_grad)
                global_norm = opt.grad_norm(fp64_norm)
            return local, global_norm, torch.ones((), device=opt.flat_grad.device)
        if self.transport == "peer" and opt.flat_grad.is_cuda:
            one = torch.ones((), device=opt.flat_grad.device)
            norm = self._peer_engine(opt).all_reduce_mean(opt.flat_grad, one)
        else:
            self._all_reduce_mean(opt.flat_grad)
            norm = opt.grad_norm(fp64_norm)
        return norm, None, coef(norm)

    def _all_reduce_mean(self, flat: torch.Tensor) -> None:
        if self.info.backend == "nccl":
            dist.all_reduce(flat, op=dist.ReduceOp.AVG)
        else:
            dist.all_reduce(flat, op=dist.ReduceOp.SUM)
            flat.div_(self.info.world_size)

    @torch.no_grad()
    def broadcast_parameters(self, opt) -> None:
        """Rank 0's parameters (and EMA shadow) to every rank, as DDP does at wrap time."""
        if not self.info.is_distributed:
            return
        dist.broadcast(opt.flat_param, src=0)
        if opt.shadow is not None:
            dist.broadcast(opt.shadow, src=0)
        if getattr(opt, "z", None) is not None:  # schedule-free: the second sequence starts from the same point
            opt.reseed_z()
        opt.refresh_bf16()
