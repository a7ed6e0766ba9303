"""Gradient all-reduce through NVLink peer memory (``ops/csrc/peer_reduce.cu``).

``PeerReducer`` moves the optimizer's flat gradient into symmetric memory
(``torch.distributed._symmetric_memory``: one allocation per rank, every rank
mapped into every other rank's address space), after which a reduction is two
launches of our own kernels and no NCCL call:

1. each rank writes its clip coefficient into its control block; a symmetric
   memory barrier makes "gradients and coefficients are final" known to all;
2. ``peer_allreduce_mean`` sums this rank's slice over all ranks with peer
   loads (scaled per source rank), averages, accumulates the squared norm and
   stores the slice into every rank's buffer with peer stores, then publishes
   the partial norm and a sequence flag; a one-warp kernel waits, bounded, for
   all flags and writes the global norm.

The kernels use plain peer loads and stores (no NVLS multicast), so a rank that
left between steps cannot fault the others; a wait that runs out reports
through the status word, returns a NaN norm and the step is skipped.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .dist import DistInfo

CTRL_BYTES = 512


class PeerReducer:
    def __init__(self, info: DistInfo, opt):
        import torch.distributed._symmetric_memory as symm_mem

        from ..ops import native

        native.require()
        self.info = info
        group = dist.group.WORLD
        try:  # older releases want the group registered first
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:  # noqa: BLE001
            pass
        dev = info.device
        n = opt.flat_grad.numel()
        if n % 4:
            raise ValueError("flat gradient length must be a multiple of 4")
        self.grad = symm_mem.empty(n, dtype=torch.float32, device=dev)
        self.ctrl = symm_mem.empty(CTRL_BYTES // 4, dtype=torch.float32, device=dev)
        self.ctrl.zero_()
        self.grad.copy_(opt.flat_grad)
        self._h_grad = symm_mem.rendezvous(self.grad, group)
        self._h_ctrl = symm_mem.rendezvous(self.ctrl, group)
        self.grad_ptrs = [int(p) for p in self._h_grad.buffer_ptrs]
        self.ctrl_ptrs = [int(p) for p in self._h_ctrl.buffer_ptrs]
        self.scratch = torch.zeros(4, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seq = 0
        # the optimizer and every parameter's .grad now live in the symmetric buffer
        opt.flat_grad = self.grad
        for i, p in enumerate(opt.params):
            p.grad = opt._view(self.grad, i)
        self._h_ctrl.barrier(channel=0)

    @torch.no_grad()
    def all_reduce_mean(self, flat_grad: torch.Tensor, coef: torch.Tensor) -> torch.Tensor:
        """``flat_grad := mean_r(coef_r * flat_grad_r)`` on every rank; returns the norm of the result."""
        if flat_grad.data_ptr() != self.grad.data_ptr():
            raise RuntimeError("PeerReducer: the optimizer's gradient buffer was replaced after adoption")
        self.ctrl[0:1].copy_(coef.reshape(1).to(torch.float32))
        self._h_ctrl.barrier(channel=0)  # every rank's backward and coefficient are done
        self.seq += 1
        return torch.ops.df3.peer_allreduce_mean(self.grad, self.grad_ptrs, self.ctrl_ptrs, self.scratch, self.status,
                                                 self.info.rank, self.info.world_size, self.seq)  # fmt: skip

    def check(self) -> None:
        """Raise if a flag wait ran out since the last check (reads the status word: synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer gradient reduction: a wait for another rank's flag timed out (status {code})")
