"""Row-tiled application of a module to very long inputs (reference: model/tiled_linear.py:37-190).

``TiledLinear(inner)`` keeps ``inner``'s parameter names (its state-dict keys are those of ``inner``) and applies it
to ``num_shards`` slices of the leading rows, so the intermediate of a wide transition never exists for all rows at
once. With ``num_shards = 0`` the count is chosen so that a slice holds at most 64 Mi elements.
"""

from __future__ import annotations

import torch
import torch.nn as nn


def auto_shards(x: torch.Tensor, budget_elems: int = 64 * 1024 * 1024) -> int:
    return max(1, -(-x.numel() // budget_elems))


def tiled_forward(x: torch.Tensor, module: nn.Module, num_shards: int, *extra) -> torch.Tensor:
    if num_shards <= 1:
        return module(x, *extra)
    lead = x.shape[0] if x.dim() > 2 else 1
    if x.dim() <= 2 or lead < num_shards:
        flat = x.reshape(-1, x.shape[-1])
        outs = [module(c, *[e.reshape(-1, e.shape[-1])[i : i + c.shape[0]] if isinstance(e, torch.Tensor) else e for e in extra])
                for i, c in ((s, flat[s : s + -(-flat.shape[0] // num_shards)]) for s in range(0, flat.shape[0], -(-flat.shape[0] // num_shards)))]  # fmt: skip
        out = torch.cat(outs, 0)
        return out.reshape(*x.shape[:-1], out.shape[-1])
    step = -(-lead // num_shards)
    return torch.cat([module(x[s : s + step], *[e[s : s + step] if isinstance(e, torch.Tensor) and e.shape[0] == lead else e for e in extra])
                      for s in range(0, lead, step)], 0)  # fmt: skip


class TiledLinear(nn.Module):
    def __init__(self, inner: nn.Module, num_shards: int = 0, tile_inference: bool = False):
        super().__init__()
        self.inner, self.num_shards, self.tile_inference = inner, num_shards, tile_inference

    def forward(self, x, *extra):
        if not self.training and not self.tile_inference:
            return self.inner(x, *extra)
        return tiled_forward(x, self.inner, self.num_shards or auto_shards(x), *extra)

    # state-dict transparency: keys are the inner module's
    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        return self.inner.state_dict(*args, destination=destination, prefix=prefix, keep_vars=keep_vars)

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        for k in list(state_dict):
            if k.startswith(prefix) and not k.startswith(prefix + "inner."):
                state_dict[prefix + "inner." + k[len(prefix) :]] = state_dict.pop(k)
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
