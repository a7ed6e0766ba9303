"""Stability probe of the Pairformer's single track (reference: training/single_track_probe.py:29-167).

On a probed step every ``PairFormerBlock`` reports the single representation ``s`` before its transition, the raw
transition output ``u`` and the residual gain ``gamma``; the probe appends one JSON line with depth statistics of
``rms(s)``, ``rms(u)``, ``rms(gamma u)``, ``cos(s, u)`` and ``alpha = <s, u> / |s|^2`` (the radial gain coefficient:
one forward grows ``|s|`` by about ``exp(sum_k gamma_k alpha_k)`` when updates align with the stream).

Statistics are accumulated as device tensors and read back once in ``end_step``, so a probed step costs one host
synchronisation instead of several per block.
"""

from __future__ import annotations

import json
import os

import torch
import torch.nn as nn

_KEYS = ("rms_s", "rms_u", "rms_gu", "cos_su", "alpha_su")


class SingleTrackProbe:
    def __init__(self, model: nn.Module, log_path: str):
        self.log_path = str(log_path)
        os.makedirs(os.path.dirname(os.path.abspath(self.log_path)), exist_ok=True)
        model = getattr(model, "module", model)
        self.blocks = list(model.evoformer.trunk_pairformer) if hasattr(model.evoformer, "trunk_pairformer") else [
            m for m in model.evoformer.modules() if type(m).__name__ == "PairFormerBlock" and getattr(m, "use_single_track", False)]  # fmt: skip
        for i, blk in enumerate(self.blocks):
            blk._probe, blk._probe_layer_idx = self, i
        self.enabled = False
        self._rows: dict[int, torch.Tensor] = {}
        self._gamma: dict[int, float] = {}
        self._step: int | None = None

    def begin_step(self, target_step: int) -> None:
        self._rows, self._gamma, self._step, self.enabled = {}, {}, int(target_step), True

    @torch.no_grad()
    def record_block(self, layer_idx: int, single_in: torch.Tensor, u: torch.Tensor, gamma) -> None:
        s, v = single_in.detach().float(), u.detach().float()
        g = float(gamma.value if hasattr(gamma, "value") else gamma)
        dot = (s * v).sum(-1)
        s2 = s.pow(2).sum(-1)
        cos = dot / (s2.sqrt().clamp_min(1e-8) * v.norm(dim=-1).clamp_min(1e-8))
        self._rows[int(layer_idx)] = torch.stack([s.pow(2).mean().sqrt(), v.pow(2).mean().sqrt(), (g * v).pow(2).mean().sqrt(),
                                                  cos.mean(), (dot / s2.clamp_min(1e-8)).mean()])  # fmt: skip
        self._gamma[int(layer_idx)] = g

    def _weight_norms(self) -> dict[str, float]:
        out = {}
        for tag, idx in (("l0", 0), ("l_mid", len(self.blocks) // 2), ("l_last", len(self.blocks) - 1)):
            if 0 <= idx < len(self.blocks) and hasattr(self.blocks[idx], "single_transition"):
                sq = sum(float(p.detach().float().pow(2).sum()) for p in self.blocks[idx].single_transition.parameters())
                out[f"w_norm_single_transition_{tag}"] = sq**0.5
        return out

    @torch.no_grad()
    def end_step(self, extra: dict | None = None) -> None:
        if not self.enabled:
            return
        self.enabled = False
        if not self._rows:
            return
        layers = sorted(self._rows)
        table = torch.stack([self._rows[i] for i in layers]).cpu()  # the one read-back of the step
        L = len(self.blocks)
        out: dict = {"step": self._step, **(extra or {})}
        pos = {layer: r for r, layer in enumerate(layers)}
        for c, key in enumerate(_KEYS):
            col = table[:, c]
            out[f"{key}_mean"], out[f"{key}_min"], out[f"{key}_max"] = float(col.mean()), float(col.min()), float(col.max())
            for tag, layer in (("l0", 0), ("l_mid", L // 2), ("l_last", L - 1)):
                out[f"{key}_{tag}"] = float(col[pos[layer]]) if layer in pos else None
        ga = [self._gamma[i] * float(table[pos[i], 4]) for i in layers]
        out["sum_gamma_alpha"], out["max_gamma_alpha"] = float(sum(ga)), float(max(ga, key=abs))
        out.update(self._weight_norms())
        with open(self.log_path, "a") as f:
            f.write(json.dumps(out) + "\n")
        self._rows = {}

    def discard_step(self) -> None:
        self.enabled, self._rows = False, {}
