"""Weight files -> a ready model (reference: scripts/_common.py:54-256).

Accepted: ``.safetensors`` (with the ``model_cfg_json`` metadata the exporter embeds), ``.pt``
training checkpoints (a snapshot is chosen with ``snapshot``) and no file at all (random weights, for
benchmarks and tests).

Snapshots of a ``.pt`` checkpoint: ``average`` = ``ckpt["model"]``; ``shadow`` = the EMA shadow laid over
it; ``fast`` = the schedule-free optimizer's ``z`` iterate; ``auto`` = shadow if the checkpoint has one,
else average.
"""

from __future__ import annotations

import logging

import torch

from ..compat import torch_load_compat

from ..config.schema import ModelConfig, OptimConfig
from ..training.checkpointing import load_safetensors, strip_module_prefix

logger = logging.getLogger(__name__)


def select_snapshot(ckpt: dict, choice: str = "auto") -> dict:
    state = dict(strip_module_prefix(ckpt["model"]))
    ema = ckpt.get("ema") or {}
    shadow = ema.get("shadow") if isinstance(ema, dict) else None
    if choice == "auto":
        choice = "shadow" if shadow else "average"
    if choice == "average":
        return state
    if choice == "shadow":
        if not shadow:
            raise ValueError("--snapshot shadow: the checkpoint has no EMA shadow")
        state.update(strip_module_prefix(shadow))
        return state
    if choice == "fast":
        names = ckpt.get("optimizer_param_names")
        opt_state = (ckpt.get("optimizer") or {}).get("state", {})
        z = {int(k): v["z"] for k, v in opt_state.items() if isinstance(v, dict) and "z" in v}
        if not z or not names:
            raise ValueError("--snapshot fast: the checkpoint has no schedule-free 'z' state")
        for idx, t in z.items():
            name = names[idx]
            if name in state and state[name].shape == t.shape:
                state[name] = t
        return state
    raise ValueError(f"unknown snapshot {choice!r}")


def load_state(path: str, snapshot: str = "auto"):
    """``(state_dict, ModelConfig or None)`` from a weight file."""
    if path.endswith(".safetensors"):
        return load_safetensors(path)
    if path.endswith((".pt", ".pth", ".ckpt")):
        ckpt = torch_load_compat(path, map_location="cpu", weights_only=False, mmap=True)
        if isinstance(ckpt, dict) and "model" in ckpt:
            return select_snapshot(ckpt, snapshot), ckpt.get("model_cfg")
        return strip_module_prefix(ckpt), None
    if path.endswith((".bin", ".bin.zst", ".zst")):
        from ..convert.af3 import convert_file

        return convert_file(path), None
    raise ValueError(f"unrecognised weight file {path!r}")


def check_loaded_keys(missing, unexpected, allow_missing: bool = False) -> None:
    markers = OptimConfig.FUSED_STATE_DICT_MARKERS
    missing = [k for k in missing if not any(m in k for m in markers)]
    unexpected = [k for k in unexpected if not any(m in k for m in markers)]
    if unexpected:
        logger.warning("%d unexpected keys in the weight file (first: %s)", len(unexpected), unexpected[:3])
    if missing and not allow_missing:
        raise RuntimeError(f"{len(missing)} parameters are missing from the weight file (first: {missing[:5]}); "
                           "pass --allow-missing-keys to run anyway")  # fmt: skip


def build_model(params: str | None, device, optim: str = "inference", snapshot: str = "auto",
                model_cfg: ModelConfig | None = None, allow_missing: bool = False):  # fmt: skip
    """Model in eval mode on ``device`` with the weights of ``params`` (random if ``None``)."""
    from ..models.model import DeepFold3

    state, file_cfg = (None, None) if params is None else load_state(params, snapshot)
    cfg = model_cfg or file_cfg or ModelConfig()
    cfg.optim = OptimConfig.from_preset(optim, getattr(file_cfg, "optim", None)) if isinstance(optim, str) else optim
    model = DeepFold3(cfg)
    if state is not None:
        res = model.load_state_dict(state, strict=False)
        check_loaded_keys(res.missing_keys, res.unexpected_keys, allow_missing)
    return model.to(device).eval(), cfg
