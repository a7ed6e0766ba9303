"""Compact storage of head logits (reference: io/logit_codec.py:58-363).

Schemes: ``f16`` (half precision), ``u8`` (per-position affine 8-bit: each logit vector is clipped to
``[max - clip, max]`` and quantised to 256 levels; softmax-relevant structure survives, 4x smaller than
fp32) and ``f32``. A file is an ``.npz`` with one payload (plus offsets for ``u8``) per head and a JSON
attribute blob.
"""

from __future__ import annotations

import dataclasses
import json

import numpy as np

DEFAULT_CLIP = 30.0
SCHEMES = ("f16", "u8", "f32")


@dataclasses.dataclass
class DecodedLogits:
    arrays: dict
    attrs: dict

    def __getitem__(self, name):
        return self.arrays[name]


def _encode(arr: np.ndarray, scheme: str, clip: float):
    arr = np.asarray(arr, dtype=np.float32)
    if scheme == "f32":
        return {"payload": arr}
    if scheme == "f16":
        return {"payload": arr.astype(np.float16)}
    if scheme == "u8":
        top = arr.max(-1, keepdims=True)
        q = np.clip((arr - (top - clip)) / clip, 0.0, 1.0)
        return {"payload": np.round(q * 255).astype(np.uint8), "top": top.astype(np.float16)}
    raise ValueError(f"unknown logit scheme {scheme!r}; choose from {SCHEMES}")


def _decode(parts: dict, scheme: str, clip: float) -> np.ndarray:
    if scheme in ("f32", "f16"):
        return parts["payload"].astype(np.float32)
    top = parts["top"].astype(np.float32)
    return top - clip + parts["payload"].astype(np.float32) / 255.0 * clip


def save_logits(path, heads: dict, scheme: str = "f16", clip: float = DEFAULT_CLIP, attrs: dict | None = None) -> None:
    blob = {}
    for name, arr in heads.items():
        if hasattr(arr, "detach"):
            arr = arr.detach().float().cpu().numpy()
        for part, val in _encode(arr, scheme, clip).items():
            blob[f"{name}.{part}"] = val
    meta = {"scheme": scheme, "clip": clip, "heads": list(heads), **(attrs or {})}
    np.savez_compressed(path, __attrs__=np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8), **blob)


def load_attrs(path) -> dict:
    with np.load(path) as z:
        return json.loads(bytes(z["__attrs__"]).decode())


def head_names(path) -> list[str]:
    return list(load_attrs(path)["heads"])


def load_logits(path) -> DecodedLogits:
    with np.load(path) as z:
        attrs = json.loads(bytes(z["__attrs__"]).decode())
        arrays = {}
        for name in attrs["heads"]:
            parts = {k.split(".", 1)[1]: z[k] for k in z.files if k.startswith(name + ".")}
            arrays[name] = _decode(parts, attrs["scheme"], attrs["clip"])
    return DecodedLogits(arrays, attrs)


def softmax(x: np.ndarray, axis: int = -1) -> np.ndarray:
    e = np.exp(x - x.max(axis, keepdims=True))
    return e / e.sum(axis, keepdims=True)


def expectation(logits: np.ndarray, centers: np.ndarray) -> np.ndarray:
    return (softmax(logits) * centers).sum(-1)


def entropy(logits: np.ndarray, axis: int = -1) -> np.ndarray:
    p = softmax(logits, axis)
    return -(p * np.log(np.clip(p, 1e-12, None))).sum(axis)


def measure_recovery(original: np.ndarray, scheme: str, clip: float = DEFAULT_CLIP) -> dict:
    """Worst and mean absolute change of the softmax probabilities after an encode / decode round trip."""
    back = _decode(_encode(original, scheme, clip), scheme, clip)
    d = np.abs(softmax(np.asarray(original, np.float32)) - softmax(back))
    return {"max_prob_err": float(d.max()), "mean_prob_err": float(d.mean())}
