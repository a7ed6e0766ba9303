"""Compact storage of head logits, in the reference's file format (io/logit_codec.py:48-363).

A file is one ``.npz``: a payload array per head under the head's own name (``distogram``, ``pae``, ``plddt``, ``pde``,
and any further head such as ``exp_resolved``), optional verbatim ``extra`` arrays, and ``_meta``: UTF-8 JSON
``{"heads": {name: {"scheme", "dtype", "shape", "scale"?, "zero_point"?, "clip"?, "bin_axis"?}}, "attrs": {...},
"version": 1}``. Files written here load in the reference and the other way round.

Schemes (the bin axis is the last one):

``float32`` / ``float16``   the logits as they are / in half precision.
``int8``                    one affine map of the whole array's [min, max] onto -128 .. 127.
``int8_softmax``            the default: every logit vector minus its maximum (softmax does not see the shift),
                            clipped to ``[-clip, 0]`` and spread over 256 levels; ``exp(-clip)`` bounds what the clip loses.
``int4_softmax``            the same over 16 levels, two values per byte along the bin axis.

The short names of earlier files (``f32``, ``f16``, ``u8``) are accepted as aliases, and files in the earlier layout
(an ``__attrs__`` blob with ``<head>.payload`` arrays) still load.
"""

from __future__ import annotations

import dataclasses
import json
import os

import numpy as np

HEADS = ("distogram", "pae", "plddt", "pde")
SCHEMES = ("float32", "float16", "int8", "int8_softmax", "int4_softmax")
ALIASES = {"f32": "float32", "f16": "float16", "u8": "int8_softmax"}
DEFAULT_CLIP = 16.0
FORMAT_VERSION = 1
_LEVELS = {"int8_softmax": 256, "int4_softmax": 16}


def canonical_scheme(scheme: str) -> str:
    name = ALIASES.get(scheme, scheme)
    if name not in SCHEMES:
        raise ValueError(f"unknown logit scheme {scheme!r}; choose from {SCHEMES} (or {tuple(ALIASES)})")
    return name


@dataclasses.dataclass
class DecodedLogits:
    heads: dict = dataclasses.field(default_factory=dict)
    extra: dict = dataclasses.field(default_factory=dict)
    attrs: dict = dataclasses.field(default_factory=dict)

    @property
    def arrays(self) -> dict:
        return self.heads

    def __getitem__(self, name):
        return self.heads[name] if name in self.heads else self.extra[name]

    def __contains__(self, name) -> bool:
        return name in self.heads or name in self.extra


def _numpy(arr) -> np.ndarray:
    if hasattr(arr, "detach"):
        arr = arr.detach().float().cpu().numpy()
    return np.asarray(arr)


def encode(arr, scheme: str, clip: float = DEFAULT_CLIP) -> tuple[np.ndarray, dict]:
    """``(payload, meta)`` of one head."""
    scheme = canonical_scheme(scheme)
    arr = _numpy(arr)
    meta = {"scheme": scheme, "dtype": arr.dtype.name, "shape": [int(d) for d in arr.shape]}
    x = arr.astype(np.float32, copy=False)
    if scheme == "float32":
        return x, meta
    if scheme == "float16":
        return x.astype(np.float16), meta
    if scheme == "int8":
        lo, hi = (float(x.min()), float(x.max())) if x.size else (0.0, 1.0)
        step = ((hi - lo) or 1.0) / 255.0
        zero = int(round(-lo / step)) - 128
        q = np.clip(np.rint(x / step).astype(np.int64) + zero, -128, 127).astype(np.int8)
        return q, {**meta, "scale": step, "zero_point": zero}
    levels = _LEVELS[scheme]
    axis = x.ndim - 1
    step = clip / (levels - 1)
    q = np.rint((np.clip(x - x.max(axis=axis, keepdims=True), -clip, 0.0) + clip) / step)
    q = np.clip(q, 0, levels - 1).astype(np.uint8)
    if scheme == "int4_softmax":
        if q.shape[axis] % 2:
            q = np.concatenate([q, np.zeros((*q.shape[:-1], 1), np.uint8)], axis=axis)
        q = (q[..., 1::2] << 4) | (q[..., 0::2] & 0x0F)  # even bins in the low nibble
    return q, {**meta, "scale": float(step), "clip": float(clip), "bin_axis": axis}


def decode(payload: np.ndarray, meta: dict) -> np.ndarray:
    scheme = canonical_scheme(meta["scheme"])
    if scheme in ("float32", "float16"):
        return payload.astype(np.float32)
    if scheme == "int8":
        return ((payload.astype(np.int32) - int(meta["zero_point"])) * float(meta["scale"])).astype(np.float32)
    q = payload.astype(np.uint8)
    if scheme == "int4_softmax":
        both = np.stack([q & 0x0F, q >> 4], axis=-1).reshape(*q.shape[:-1], -1)
        q = both[..., : int(meta["shape"][-1])]
    # the row maxima are gone, which softmax does not notice: the result is the logits minus their row maximum
    return q.astype(np.float32) * float(meta["scale"]) - float(meta["clip"])


def save_logits(path, heads: dict | None = None, scheme: str = "int8_softmax", clip: float = DEFAULT_CLIP, attrs: dict | None = None,
                *, extra: dict | None = None, **named_heads) -> None:  # fmt: skip
    """Write the given heads (a dict, and / or keyword arguments ``distogram=``, ``pae=``, ``plddt=``, ``pde=``, ...;
    ``None`` values are skipped) with one scheme. ``extra`` arrays are stored verbatim, ``attrs`` inside ``_meta``."""
    scheme = canonical_scheme(scheme)
    arrays, metas = {}, {}
    for name, arr in {**(heads or {}), **named_heads}.items():
        if arr is None:
            continue
        arrays[name], metas[name] = encode(arr, scheme, clip)
    for name, arr in (extra or {}).items():
        if name in metas or name == "_meta":
            raise ValueError(f"extra array {name!r} collides with a head or a reserved name")
        arrays[name] = _numpy(arr)
    blob = json.dumps({"heads": metas, "attrs": attrs or {}, "version": FORMAT_VERSION}).encode("utf-8")
    arrays["_meta"] = np.frombuffer(blob, dtype=np.uint8)
    os.makedirs(os.path.dirname(os.path.abspath(str(path))), exist_ok=True)
    np.savez_compressed(path, **arrays)


def _meta_of(z) -> dict:
    return json.loads(bytes(z["_meta"]).decode("utf-8"))


def load_attrs(path) -> dict:
    """Only the attribute dict (seed, sample index, bin edges, ...): no payload is decoded."""
    with np.load(path) as z:
        if "_meta" in z.files:
            return _meta_of(z).get("attrs", {})
        return json.loads(bytes(z["__attrs__"]).decode())


def head_names(path) -> list[str]:
    with np.load(path) as z:
        if "_meta" in z.files:
            return list(_meta_of(z)["heads"])
        return list(json.loads(bytes(z["__attrs__"]).decode())["heads"])


def _load_earlier_layout(z) -> DecodedLogits:
    attrs = json.loads(bytes(z["__attrs__"]).decode())
    out = {}
    for name in attrs["heads"]:
        payload = z[f"{name}.payload"]
        if attrs["scheme"] == "u8":
            top, clip = z[f"{name}.top"].astype(np.float32), float(attrs["clip"])
            out[name] = top - clip + payload.astype(np.float32) / 255.0 * clip
        else:
            out[name] = payload.astype(np.float32)
    return DecodedLogits(out, {}, attrs)


def load_logits(path) -> DecodedLogits:
    with np.load(path) as z:
        if "_meta" not in z.files:
            return _load_earlier_layout(z)
        meta = _meta_of(z)
        if int(meta.get("version", 1)) > FORMAT_VERSION:
            raise ValueError(f"{path}: logit file version {meta['version']} is newer than this reader ({FORMAT_VERSION})")
        heads = {name: decode(z[name], m) for name, m in meta["heads"].items()}
        extra = {k: z[k] for k in z.files if k != "_meta" and k not in heads}
    return DecodedLogits(heads, extra, meta.get("attrs", {}))


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
    payload, meta = encode(original, scheme, clip)
    d = np.abs(softmax(np.asarray(original, np.float32)) - softmax(decode(payload, meta)))
    return {"max_prob_err": float(d.max()), "mean_prob_err": float(d.mean())}
