"""Window-averaged metrics and CUDA-event step timing.

``DistributedAverageMeters`` accumulates on the device without syncing and
reduces across ranks only at a log boundary: one key-union gather plus one
packed float64 all-reduce (reference: training/meters.py:9-129).
``StepTimeMeter`` times micro-steps with a reusable pool of CUDA events and
reads them only at the boundary (reference: training/step_timer.py:37-130).
"""

from __future__ import annotations

import time

import torch
import torch.distributed as dist


class DistributedAverageMeters:
    def __init__(self, info):
        self.info = info
        self.sums: dict[str, torch.Tensor] = {}
        self.counts: dict[str, float] = {}

    def update(self, values: dict, counts: dict | None = None) -> None:
        for k, v in values.items():
            n = float(counts.get(k, 1)) if counts else 1.0
            v = v.detach().double() * n if torch.is_tensor(v) else torch.tensor(float(v) * n, dtype=torch.float64)
            self.sums[k] = self.sums[k] + v.to(self.sums[k].device) if k in self.sums else v
            self.counts[k] = self.counts.get(k, 0.0) + n

    def sync(self) -> dict[str, float]:
        """Cross-rank weighted means of everything accumulated since the last call; resets the window."""
        keys = sorted(self.sums)
        if self.info.is_distributed:
            gathered = [None] * self.info.world_size
            dist.all_gather_object(gathered, keys)
            keys = sorted(set().union(*gathered))
        dev = self.info.device
        packed = torch.zeros(2 * len(keys), dtype=torch.float64, device=dev)
        for i, k in enumerate(keys):
            if k in self.sums:
                packed[2 * i] = self.sums[k].to(dev)
                packed[2 * i + 1] = self.counts[k]
        if self.info.is_distributed:
            if self.info.backend == "nccl":
                dist.all_reduce(packed)
            else:
                cpu = packed.cpu()
                dist.all_reduce(cpu)
                packed = cpu
        vals = packed.tolist()
        out = {k: vals[2 * i] / vals[2 * i + 1] for i, k in enumerate(keys) if vals[2 * i + 1] > 0}
        self.sums.clear()
        self.counts.clear()
        return out


class StepTimeMeter:
    """Per-micro-step device time; ``flush`` returns ``(mean_ms, max_ms, n)`` and recycles the events."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self._pool: list = []
        self._pending: list = []
        self._wall: list[float] = []
        self._t0 = 0.0

    def start(self) -> None:
        if not self.enabled:
            self._t0 = time.perf_counter()
            return
        a = self._pool.pop() if self._pool else torch.cuda.Event(enable_timing=True)
        b = self._pool.pop() if self._pool else torch.cuda.Event(enable_timing=True)
        a.record()
        self._pending.append((a, b))

    def stop(self) -> None:
        if not self.enabled:
            self._wall.append((time.perf_counter() - self._t0) * 1e3)
            return
        self._pending[-1][1].record()

    def flush(self):
        if self.enabled:
            if self._pending:
                self._pending[-1][1].synchronize()
            ms = [a.elapsed_time(b) for a, b in self._pending]
            for a, b in self._pending:
                self._pool += [a, b]
            self._pending.clear()
        else:
            ms, self._wall = self._wall, []
        if not ms:
            return 0.0, 0.0, 0
        return sum(ms) / len(ms), max(ms), len(ms)
