"""Data-parallel gradient path through NVLink peer memory (``ops/csrc/peer_reduce.cu``).

Every rank's flat fp32 gradient and a 1 KiB control block live in device memory that all ranks of the node map into
their address space. The mapping is set up once: plain device allocations are exported as CUDA IPC handles, the
handles travel over the process group, and each rank opens its peers' handles (``torch.distributed`` symmetric memory
is the fallback when IPC is unavailable). After that two forms of the step run on our own kernels, with plain peer
loads and stores and no NCCL call:

``PeerReducer.all_reduce_mean``
    bounded entry arrive/wait on the control blocks, then one kernel that reduce-scatters, scales by each source
    rank's clip coefficient, averages, accumulates the squared norm and all-gathers, then a one-warp kernel that waits
    (bounded) for every rank's done flag and writes the global norm.

``PeerReducer.fused_step``
    one cooperative kernel for the whole optimizer step: entry wait, reduction, norm and flag exchange, the skip /
    clip decision taken identically on every rank from the exchanged flags, AdamW + EMA + bf16 mirror, gradient zeroing.
    The host reads the outcome later from a small result block copied back asynchronously
    (reference sequence being replaced: training/optim.py:576-765, training/ema.py:77-90).

No wait in these kernels is unbounded and none traps: a wait that runs out records a status code, the kernels leave
peer memory alone and the step counts as skipped. NVLS is not used, so a rank that left between steps
cannot fault the others.
"""

from __future__ import annotations

import logging

import torch
import torch.distributed as dist

from .dist import DistInfo

logger = logging.getLogger(__name__)
CTRL_BYTES = 1024
MAX_WORLD = 16
RESULT_FLOATS = 4 + 2 * MAX_WORLD


def _share_over_ipc(info: DistInfo, nbytes: int):
    """``(local uint8 buffer, [device address of every rank's buffer])`` through CUDA IPC handles."""
    ops = torch.ops.df3
    dev = info.device.index if info.device.index is not None else torch.cuda.current_device()
    buf = ops.peer_alloc(int(nbytes), int(dev))
    handle = ops.peer_ipc_handle(buf)
    handles = [None] * info.world_size
    dist.all_gather_object(handles, bytes(handle.numpy().tobytes()))
    ptrs = []
    for r, raw in enumerate(handles):
        if r == info.rank:
            ptrs.append(int(buf.data_ptr()))
        else:
            h = torch.frombuffer(bytearray(raw), dtype=torch.uint8).clone()
            ptrs.append(int(ops.peer_ipc_open(h, int(dev))))
    return buf, ptrs


def _share_over_symmetric_memory(info: DistInfo, nbytes: int):
    import torch.distributed._symmetric_memory as symm_mem

    buf = symm_mem.empty(int(nbytes), dtype=torch.uint8, device=info.device)
    buf.zero_()
    handle = symm_mem.rendezvous(buf, dist.group.WORLD)
    return buf, [int(p) for p in handle.buffer_ptrs], handle


class PeerReducer:
    def __init__(self, info: DistInfo, opt):
        from ..ops import native

        native.require()
        self.info = info
        dev = info.device
        n = opt.flat_grad.numel()
        if n % 4:
            raise ValueError("flat gradient length must be a multiple of 4")
        if info.world_size > MAX_WORLD:
            raise ValueError(f"peer gradient path supports up to {MAX_WORLD} ranks on one node")
        self._keep = []  # symmetric-memory handles must outlive the mappings
        self.bootstrap = "local"
        if info.world_size == 1:
            grad8 = torch.zeros(n * 4, dtype=torch.uint8, device=dev)
            ctrl8 = torch.zeros(CTRL_BYTES, dtype=torch.uint8, device=dev)
            self.grad_ptrs, self.ctrl_ptrs = [grad8.data_ptr()], [ctrl8.data_ptr()]
        else:
            try:
                grad8, self.grad_ptrs = _share_over_ipc(info, n * 4)
                ctrl8, self.ctrl_ptrs = _share_over_ipc(info, CTRL_BYTES)
                self.bootstrap = "cuda-ipc"
            except Exception as exc:  # noqa: BLE001 - the decision must be the same on every rank, see below
                grad8 = ctrl8 = None
                logger.warning("CUDA IPC sharing of the gradient buffer failed (%r)", exc)
            ok = torch.tensor([1 if grad8 is not None else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:  # some rank could not share over IPC: everybody takes symmetric memory
                grad8, self.grad_ptrs, h1 = _share_over_symmetric_memory(info, n * 4)
                ctrl8, self.ctrl_ptrs, h2 = _share_over_symmetric_memory(info, CTRL_BYTES)
                self._keep += [h1, h2]
                self.bootstrap = "symmetric-memory"
        self.grad = grad8.view(torch.float32)
        self.ctrl = ctrl8.view(torch.float32)
        self.grad.copy_(opt.flat_grad)
        self.scratch = torch.zeros(4, dtype=torch.float32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.result = torch.zeros(RESULT_FLOATS, dtype=torch.float32, device=dev)
        self.result_host = torch.zeros(RESULT_FLOATS, dtype=torch.float32).pin_memory()
        self.result_event = None
        self.seq = 0
        # the optimizer and every parameter's .grad now live in the shared buffer
        opt.flat_grad = self.grad
        for i, p in enumerate(opt.params):
            p.grad = opt._view(self.grad, i)
        if info.world_size > 1:
            torch.cuda.synchronize(dev)
            dist.barrier()  # set-up only: every rank's buffers are mapped and zeroed before the first step

    def _own(self, flat_grad: torch.Tensor) -> None:
        if flat_grad.data_ptr() != self.grad.data_ptr():
            raise RuntimeError("PeerReducer: the optimizer's gradient buffer was replaced after adoption")

    @torch.no_grad()
    def all_reduce_mean(self, flat_grad: torch.Tensor, coef: torch.Tensor, spin_limit: int = 0) -> torch.Tensor:
        """``flat_grad := mean_r(coef_r * flat_grad_r)`` on every rank; returns the norm of the result (NaN if a wait
        for another rank ran out; ``check()`` then raises)."""
        self._own(flat_grad)
        self.ctrl[0:1].copy_(coef.reshape(1).to(torch.float32))
        self.seq += 1
        return torch.ops.df3.peer_allreduce_mean(self.grad, self.grad_ptrs, self.ctrl_ptrs, self.scratch, self.status,
                                                 self.info.rank, self.info.world_size, self.seq, spin_limit)  # fmt: skip

    @torch.no_grad()
    def fused_step(self, opt, *, coef, loss_flag, local_norm, lr, betas, eps, bc1, bc2, ema, ema_w, clip_norm, skip_threshold,
                   per_rank_clip: bool, spin_limit: int = 0) -> None:  # fmt: skip
        """Launch the one-kernel optimizer step. ``coef``, ``loss_flag`` and ``local_norm`` are device scalars; the
        outcome arrives in ``result_host`` once ``result_event`` has completed (``read_result``)."""
        self._own(opt.flat_grad)
        self.ctrl[0:3].copy_(torch.stack([coef.reshape(()).float(), loss_flag.reshape(()).float(), local_norm.reshape(()).float()]))
        self.seq += 1
        torch.ops.df3.peer_fused_step(
            self.grad, self.grad_ptrs, self.ctrl_ptrs, self.scratch, self.status, self.result, opt.flat_param, opt.exp_avg,
            opt.exp_avg_sq, ema, opt.decay_vec, opt.flat_param_bf16, self.info.rank, self.info.world_size, self.seq, float(lr),
            float(betas[0]), float(betas[1]), float(eps), float(bc1), float(bc2), float(ema_w), float(clip_norm or 0.0),
            float(skip_threshold or 0.0), bool(per_rank_clip), int(spin_limit),
        )  # fmt: skip
        self.result_host.copy_(self.result, non_blocking=True)
        self.result_event = torch.cuda.Event()
        self.result_event.record()

    def read_result(self) -> dict | None:
        """Outcome of the last ``fused_step`` (waits for its copy if it has not landed yet); ``None`` if none is pending."""
        if self.result_event is None:
            return None
        self.result_event.synchronize()
        self.result_event = None
        r = self.result_host
        w = self.info.world_size
        return {"advanced": bool(r[0] > 0.5), "reason": {0: None, 1: "loss", 2: "grad", 3: "timeout"}[int(r[1])],
                "norm": float(r[2]), "scale": float(r[3]), "loss_flags": [float(x) for x in r[4 : 4 + w]],
                "local_norms": [float(x) for x in r[4 + MAX_WORLD : 4 + MAX_WORLD + w]]}  # fmt: skip

    def check(self) -> None:
        """Raise if a flag wait ran out since the last check (reads the status word: synchronises)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer gradient reduction: a wait for another rank's flag timed out (status {code})")
