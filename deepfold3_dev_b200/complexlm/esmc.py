"""Warm start of the complex language model from a released ESM-C checkpoint.

The blocks of ``ComplexLM`` follow ESM-C's design (pre-norm attention with a fused q/k/v projection and q/k LayerNorm,
SwiGLU feed-forward of ESM-C's width rule, a norm before the read-out), so with ``esmc_compat`` set every ESM-C tensor
has exactly one counterpart here and values are copied without any re-arrangement (reference: complexlm/esmc.py:1-117).
Names translate by the rules in ``RULES``; the only shape difference allowed is the vocabulary axis: ESM-C's token
table has 64 rows whose first 33 are the ESM-2 tokens in ESM-2's order, which is the vocabulary used here, so the
embedding and the read-out take the leading rows.

What does not carry over is position: ESM-C trained every layer with rotary embeddings, while the complex-scoped
layers here attend without any. Their projections and feed-forward weights are still copied; their attention pattern is
learned anew, which shows as an early loss bump concentrated in those layers.
"""

from __future__ import annotations

import logging
import re

import torch

logger = logging.getLogger(__name__)

# released sizes: the model must have exactly this shape for a tensor-for-tensor copy
ESMC_SHAPES = {"esmc-300m": {"d_model": 960, "n_layers": 30, "n_heads": 15}, "esmc-600m": {"d_model": 1152, "n_layers": 36, "n_heads": 18}}

# (pattern on the ESM-C module path, replacement giving the module path here); first match wins
RULES = (
    (r"^embed$", "embed"),
    (r"^transformer\.norm$", "norm"),
    (r"^transformer\.blocks\.(\d+)\.attn\.layernorm_qkv\.0$", r"blocks.\1.attn.norm"),
    (r"^transformer\.blocks\.(\d+)\.attn\.layernorm_qkv\.1$", r"blocks.\1.attn.qkv"),
    (r"^transformer\.blocks\.(\d+)\.attn\.q_ln$", r"blocks.\1.attn.q_norm"),
    (r"^transformer\.blocks\.(\d+)\.attn\.k_ln$", r"blocks.\1.attn.k_norm"),
    (r"^transformer\.blocks\.(\d+)\.attn\.out_proj$", r"blocks.\1.attn.out_proj"),
    (r"^transformer\.blocks\.(\d+)\.ffn\.0$", r"blocks.\1.ffn.norm"),
    (r"^transformer\.blocks\.(\d+)\.ffn\.1$", r"blocks.\1.ffn.w_in"),
    (r"^transformer\.blocks\.(\d+)\.ffn\.3$", r"blocks.\1.ffn.w_out"),
    (r"^sequence_head\.0$", "head.dense"),
    (r"^sequence_head\.2$", "head.norm"),
    (r"^sequence_head\.3$", "head.out"),
)


def translate(name: str) -> str | None:
    """Parameter name here for an ESM-C parameter name (``<module path>.weight|bias``), or ``None`` without a counterpart."""
    module, _, leaf = name.rpartition(".")
    if leaf not in ("weight", "bias"):
        return None
    for pattern, target in RULES:
        if re.match(pattern, module):
            return re.sub(pattern, target, module) + "." + leaf
    return None


def matching_release(cfg) -> str | None:
    for name, shape in ESMC_SHAPES.items():
        if all(getattr(cfg, k) == v for k, v in shape.items()):
            return name
    return None


@torch.no_grad()
def load_esmc(model, path: str, strict: bool = True) -> dict:
    """Copy the tensors of an ESM-C checkpoint (a state dict, or a dict holding one under ``state_dict``) into ``model``.

    Returns ``{"checkpoint", "copied", "left_random", "unused_source"}``. With ``strict`` a parameter of the model that
    received nothing is an error: the point of a warm start is that no tensor stays random without anyone noticing.
    """
    if not model.cfg.esmc_compat:
        raise ValueError("esmc_compat must be set: without it the model has no biases on the norms ESM-C has them on")
    blob = torch.load(path, map_location="cpu", weights_only=False)
    source = blob.get("state_dict", blob) if isinstance(blob, dict) else blob
    params = dict(model.named_parameters())
    copied, unused = [], []
    for name, value in source.items():
        target = translate(name)
        if target is None or target not in params:
            unused.append(name)
            continue
        dest = params[target]
        if value.shape != dest.shape:
            if value.dim() >= 1 and value.shape[1:] == dest.shape[1:] and value.shape[0] > dest.shape[0]:
                value = value[: dest.shape[0]]  # the vocabulary axis: ESM-C pads its table to 64 rows
            else:
                raise ValueError(f"{name} {tuple(value.shape)} does not fit {target} {tuple(dest.shape)}")
        dest.copy_(value.to(dest.dtype))
        copied.append(target)
    missing = sorted(set(params) - set(copied))
    if missing and strict:
        raise ValueError(f"{len(missing)} parameters got nothing from the ESM-C checkpoint, e.g. {missing[:6]}")
    logger.info("ESM-C warm start from %s: %d tensors copied, %d left at their initial values", path, len(copied), len(missing))
    return {"checkpoint": str(path), "copied": len(copied), "left_random": missing, "unused_source": sorted(unused)}
