"""AdamW + EMA over one flat fp32 buffer per quantity.

The reference steps ``torch.optim.AdamW(fused=True)`` over ~3.8k separate
parameter tensors, clips with a multi-tensor multiply and updates the EMA with
``_foreach_lerp_`` (training/optim.py:195-312, training/ema.py:77-90). Here
parameters, gradients, both Adam moments and the EMA shadow each live in ONE
contiguous fp32 buffer; every ``nn.Parameter`` (and its ``.grad``) is a view
into it. The whole optimizer step - gradient scaling by the clip coefficient,
decoupled weight decay, Adam moments, the update, and the EMA lerp - is then a
single pass over memory (one CUDA kernel on a GPU, a handful of whole-buffer
torch ops on CPU), and the data-parallel gradient reduction operates on one
buffer as well.

Numerics are those of ``torch.optim.AdamW`` (bias-corrected, ``eps`` added
after the square root) followed by ``shadow.lerp_(param, 1 - decay)``.
``state_dict`` / ``load_state_dict`` use the ``torch.optim.AdamW`` layout so
``.pt`` checkpoints interchange with the reference.
"""

from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..config.schema import OptimConfig

NO_DECAY_NAME_PARTS = (
    ".to_g.", ".out_gate.", ".gate.", "cond_scale.", "cond_bias.", "zero_cond.", ".embed_", "single_activations.",
    "msa_activations.", "extra_msa_target_feat.", "left_single.", "right_single.", "position_activations.",
    "bond_embedding.", "prev_embedding.", "prev_single_embedding.",
)  # fmt: skip
ALIGN = 64  # elements; every parameter starts on a 256-byte boundary inside the flat buffers


def is_no_decay(name: str, param: torch.Tensor) -> bool:
    """1-D tensors, per-channel scale-like matrices, gates, AdaLN-zero projections and input embeddings do not decay
    (reference: training/optim.py:166-193, :214-225)."""
    if param.dim() < 2 or min(param.shape) == 1:
        return True
    return name.endswith(".weight") and any(part in name for part in NO_DECAY_NAME_PARTS)


def _is_fused_marker(name: str) -> bool:
    return any(m in name for m in OptimConfig.FUSED_STATE_DICT_MARKERS)


class FlatAdamW:
    """Flat-buffer AdamW with an optional EMA shadow.

    Attributes:
        names, params: trainable parameters in ``model.named_parameters()`` order.
        flat_param / flat_grad / exp_avg / exp_avg_sq / shadow: fp32 buffers of ``numel`` elements.
        decay_vec: per-element weight-decay coefficient (0 on no-decay segments).
        param_groups: ``[{"lr", "betas", "eps", "weight_decay", "params"}]`` mirroring torch's layout:
            group 0 decayed, group 1 not decayed, further groups for ``strong_decay`` multipliers.
    """

    def __init__(self, model: nn.Module, lr=1.8e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0,
                 strong_decay: dict | None = None, ema_decay: float = 0.0):  # fmt: skip
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        if not named:
            raise ValueError("no trainable parameters")
        for n, p in named:
            if p.dtype != torch.float32:
                raise ValueError(
                    f"FlatAdamW requires fp32 master weights, got dtype={p.dtype} for {n} with shape {tuple(p.shape)}"
                )
        self.names = [n for n, _ in named]
        self.params = [p for _, p in named]
        dev = self.params[0].device
        self.device = dev
        self.offsets, total = [], 0
        for p in self.params:
            self.offsets.append(total)
            total += (p.numel() + ALIGN - 1) // ALIGN * ALIGN
        self.numel = total
        self.flat_param = torch.zeros(total, device=dev)
        self.flat_grad = torch.zeros(total, device=dev)
        self.exp_avg = torch.zeros(total, device=dev)
        self.exp_avg_sq = torch.zeros(total, device=dev)
        self.decay_vec = torch.zeros(total, device=dev)
        strong = dict(strong_decay or {})
        group_of: list[int] = []
        mults: list[float] = []
        for n, p in named:
            if is_no_decay(n, p):
                group_of.append(1)
                continue
            hit = next((m for sub, m in strong.items() if sub in n), None)
            if hit is None:
                group_of.append(0)
            else:
                if hit not in mults:
                    mults.append(hit)
                group_of.append(2 + mults.index(hit))
        self.param_groups = [
            dict(lr=lr, initial_lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, params=[]),
            dict(lr=lr, initial_lr=lr, betas=tuple(betas), eps=eps, weight_decay=0.0, params=[]),
        ] + [dict(lr=lr, initial_lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay * m, params=[]) for m in mults]
        # torch numbers parameters group by group; keep that numbering for checkpoints
        order = sorted(range(len(named)), key=lambda i: (group_of[i], i))
        self._torch_index = {}
        for k, i in enumerate(order):
            self._torch_index[i] = k
            self.param_groups[group_of[i]]["params"].append(k)
        with torch.no_grad():
            for i, p in enumerate(self.params):
                view = self._view(self.flat_param, i)
                view.copy_(p.data)
                p.data = view
                p.grad = self._view(self.flat_grad, i)
                o = self.offsets[i]
                self.decay_vec[o : o + p.numel()] = self.param_groups[group_of[i]]["weight_decay"]
        self._group_of = group_of
        # bf16 mirror of the parameters for the tensor-core kernels: refreshed by the step kernel, so the
        # forward never casts a weight
        self.flat_param_bf16 = None
        if self.flat_param.is_cuda:
            from ..ops import autograd_ops

            self.flat_param_bf16 = self.flat_param.to(torch.bfloat16)
            for i, p in enumerate(self.params):
                autograd_ops.register_bf16_mirror(p, self._view(self.flat_param_bf16, i))
        self.step_count = 0
        self.ema_decay = float(ema_decay)
        self.ema_updates = 0
        self.ema_names = [n for n in self.names if not _is_fused_marker(n)]
        self.shadow = self.flat_param.clone() if ema_decay > 0 else None
        self.state: dict = {}  # torch.optim API parity; the moments live in the flat buffers

    def _view(self, flat: torch.Tensor, i: int) -> torch.Tensor:
        p = self.params[i]
        o = self.offsets[i]
        return flat[o : o + p.numel()].view(p.shape)

    # ------------------------------------------------------------------ gradients
    def zero_grad(self, set_to_none: bool = False) -> None:
        """Zero the flat gradient and re-attach every ``.grad`` view (``set_to_none`` is ignored by design)."""
        self.flat_grad.zero_()
        for i, p in enumerate(self.params):
            if p.grad is None or p.grad.data_ptr() != self.flat_grad.data_ptr() + 4 * self.offsets[i]:
                p.grad = self._view(self.flat_grad, i)

    def grad_norm(self, fp64: bool = True) -> torch.Tensor:
        """Global L2 norm of the flat gradient (padding is zero), fp32 scalar."""
        if fp64:
            return torch.linalg.vector_norm(self.flat_grad, 2, dtype=torch.float64).to(torch.float32)
        return torch.linalg.vector_norm(self.flat_grad, 2)

    # ------------------------------------------------------------------ step
    @torch.no_grad()
    def step(self, grad_scale: torch.Tensor | float = 1.0, update_ema: bool = True) -> None:
        """One AdamW step with every gradient multiplied by ``grad_scale`` first, then the EMA update."""
        self.step_count += 1
        g0 = self.param_groups[0]
        lr, (b1, b2), eps = g0["lr"], g0["betas"], g0["eps"]
        bc1 = 1.0 - b1**self.step_count
        bc2 = 1.0 - b2**self.step_count
        ema = self.shadow if (update_ema and self.shadow is not None) else None
        if ema is not None:
            self.ema_updates += 1
        if self.flat_param.is_cuda:
            from ..ops import native

            nat = native.require()
            if nat.has("adamw_ema"):
                scale = grad_scale if torch.is_tensor(grad_scale) else torch.tensor(float(grad_scale), device=self.device)
                nat.adamw_ema_flat(
                    self.flat_param, self.flat_grad, self.exp_avg, self.exp_avg_sq, ema, self.decay_vec,
                    scale.reshape(1).float(), lr, b1, b2, eps, bc1, bc2, 1.0 - self.ema_decay, self.flat_param_bf16,
                )  # fmt: skip
                return
        g = self.flat_grad * grad_scale
        if any(grp["weight_decay"] != 0.0 for grp in self.param_groups):
            self.flat_param.mul_(1.0 - lr * self.decay_vec)
        self.exp_avg.lerp_(g, 1.0 - b1)
        self.exp_avg_sq.mul_(b2).addcmul_(g, g, value=1.0 - b2)
        denom = (self.exp_avg_sq.sqrt() / math.sqrt(bc2)).add_(eps)
        self.flat_param.addcdiv_(self.exp_avg, denom, value=-lr / bc1)
        if ema is not None:
            ema.lerp_(self.flat_param, 1.0 - self.ema_decay)
        self.refresh_bf16()

    @torch.no_grad()
    def refresh_bf16(self) -> None:
        """Re-derive the bf16 mirror and drop cached weight copies after the parameters were written in place."""
        if self.flat_param_bf16 is not None:
            from ..ops import autograd_ops

            self.flat_param_bf16.copy_(self.flat_param)
            autograd_ops.invalidate_weight_cache()

    def set_lr(self, lr: float) -> None:
        for g in self.param_groups:
            g["lr"] = lr

    # ------------------------------------------------------------------ EMA (reference: training/ema.py)
    def ema_state_dict(self) -> dict:
        shadow = {}
        if self.shadow is not None:
            keep = set(self.ema_names)
            for i, n in enumerate(self.names):
                if n in keep:
                    shadow[n] = self._view(self.shadow, i).clone()
        return {"decay": self.ema_decay, "num_updates": self.ema_updates, "shadow": shadow}

    @torch.no_grad()
    def load_ema_state_dict(self, state: dict) -> None:
        self.ema_decay = state["decay"]
        self.ema_updates = state["num_updates"]
        if self.shadow is None:
            self.shadow = self.flat_param.clone()
        for i, n in enumerate(self.names):
            if n in state["shadow"]:
                self._view(self.shadow, i).copy_(state["shadow"][n])

    @torch.no_grad()
    def ema_reseed(self) -> None:
        """Shadow := current parameters (resume from a checkpoint that carries no shadow)."""
        if self.shadow is not None:
            self.shadow.copy_(self.flat_param)

    def ema_swap(self) -> None:
        """Exchange live parameters and shadow in place (call again to restore)."""
        if self.shadow is None:
            return
        with torch.no_grad():
            tmp = self.flat_param.clone()
            self.flat_param.copy_(self.shadow)
            self.shadow.copy_(tmp)
        self.refresh_bf16()

    # ------------------------------------------------------------------ torch.optim.AdamW checkpoint layout
    def state_dict(self) -> dict:
        state = {}
        if self.step_count > 0:
            for i in range(len(self.params)):
                state[self._torch_index[i]] = {
                    "step": torch.tensor(float(self.step_count)),
                    "exp_avg": self._view(self.exp_avg, i).clone(),
                    "exp_avg_sq": self._view(self.exp_avg_sq, i).clone(),
                }
        groups = [{**{k: v for k, v in g.items() if k != "params"}, "amsgrad": False, "maximize": False,
                   "foreach": None, "capturable": False, "differentiable": False, "fused": None,
                   "decoupled_weight_decay": True, "params": list(g["params"])} for g in self.param_groups]  # fmt: skip
        return {"state": state, "param_groups": groups}

    @torch.no_grad()
    def load_state_dict(self, sd: dict) -> None:
        inv = {k: i for i, k in self._torch_index.items()}
        steps = set()
        for k, st in sd.get("state", {}).items():
            i = inv[int(k)]
            for key, buf in (("exp_avg", self.exp_avg), ("exp_avg_sq", self.exp_avg_sq)):
                t = st[key]
                if t.dtype != torch.float32:
                    raise ValueError(f"AdamW state['{key}'] must be fp32, got {t.dtype}")
                self._view(buf, i).copy_(t)
            steps.add(int(float(st["step"])))
        if steps:
            self.step_count = max(steps)
        for mine, theirs in zip(self.param_groups, sd.get("param_groups", [])):
            for key in ("lr", "initial_lr", "betas", "eps", "weight_decay"):
                if key in theirs:
                    mine[key] = tuple(theirs[key]) if key == "betas" else theirs[key]
        for i, p in enumerate(self.params):  # weight decay may have changed with the loaded groups
            o = self.offsets[i]
            self.decay_vec[o : o + p.numel()] = self.param_groups[self._group_of[i]]["weight_decay"]

    def param_names_by_index(self) -> list[str]:
        """Name of parameter ``k`` in the checkpoint numbering (the blob's ``optimizer_param_names``)."""
        out = [""] * len(self.params)
        for i, k in self._torch_index.items():
            out[k] = self.names[i]
        return out
