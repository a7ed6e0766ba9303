"""RMS of the residual stream and of every branch output per Pairformer layer
(reference: training/activation_meter.py:63-256).

The blocks call ``record_all_branches`` / ``record_branch`` when a meter is attached and enabled. Values are
accumulated on the device (sum of squares and element counts per layer and branch, no sync) and read once
in ``flush_to_dict``.
"""

from __future__ import annotations

import torch
import torch.nn as nn

BRANCHES = ("b_tri_out", "b_tri_in", "b_pair_attn_row", "b_pair_attn_col", "b_pair_ffn", "b_single_attn", "b_single_ffn",
            "single", "pair")  # fmt: skip


class ActivationRMSMeter:
    def __init__(self, num_layers: int, device):
        self.num_layers, self.device, self.enabled = num_layers, device, False
        self.reset()

    def reset(self) -> None:
        self.sumsq = torch.zeros(self.num_layers, len(BRANCHES), device=self.device, dtype=torch.float64)
        self.count = torch.zeros(self.num_layers, len(BRANCHES), device=self.device, dtype=torch.float64)

    @torch.no_grad()
    def _add(self, layer: int, name: str, t) -> None:
        if not isinstance(t, torch.Tensor) or t.numel() <= 1:
            return
        j = BRANCHES.index(name)
        self.sumsq[layer, j] += t.detach().float().pow(2).sum().double()
        self.count[layer, j] += t.numel()

    def record_all_branches(self, layer: int, **branches) -> None:
        for name, t in branches.items():
            self._add(layer, name, t)

    def record(self, point: int, single, pair) -> None:
        """Residual stream after ``point`` blocks (0 = after the MSA stack)."""
        if self.enabled and point > 0:
            self.record_branch(point - 1, single, pair)

    def record_branch(self, layer: int, single_delta, pair_delta) -> None:
        self._add(layer, "single", single_delta)
        self._add(layer, "pair", pair_delta)

    def flush_to_dict(self, prefix: str = "act_rms", all_ranks: bool = True) -> dict[str, float]:
        """Window statistics as log entries. In a multi-process run the sums of squares and counts are added over the
        ranks first (one all-reduce of two small tensors), so the logged RMS describes the global batch and every
        rank reports the same numbers (reference: training/activation_meter.py, its cross-rank reduction)."""
        sumsq, count = self.sumsq, self.count
        if all_ranks and torch.distributed.is_available() and torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
            both = torch.stack([sumsq.double(), count.double()])
            torch.distributed.all_reduce(both)
            sumsq, count = both[0], both[1]
        rms = (sumsq / count.clamp(min=1)).sqrt().cpu()
        seen = (count > 0).cpu()
        out = {}
        for j, name in enumerate(BRANCHES):
            vals = [float(rms[i, j]) for i in range(self.num_layers) if seen[i, j]]
            if vals:
                out[f"{prefix}/{name}_mean"] = sum(vals) / len(vals)
                out[f"{prefix}/{name}_max"] = max(vals)
                out[f"{prefix}/{name}_last"] = vals[-1]
        self.reset()
        return out


def attach_activation_meter(model: nn.Module, device) -> ActivationRMSMeter:
    """Give every Pairformer block of ``model`` a shared meter and its layer index."""
    from ..models.evoformer import PairFormerBlock

    blocks = [m for m in model.modules() if isinstance(m, PairFormerBlock)]
    meter = ActivationRMSMeter(max(1, len(blocks)), device)
    for i, b in enumerate(blocks):
        b._act_meter, b._act_layer_idx = meter, i
    for m in model.modules():
        if hasattr(m, "_grad_checkpoint") and hasattr(m, "pairformer"):
            m._act_meter = meter
    return meter
