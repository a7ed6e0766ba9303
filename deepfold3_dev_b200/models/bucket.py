"""Token-count buckets (reference: model/bucket.py:22-228).

Kernels here have no shape-specialised compilation step, but fixed shapes still pay: CUDA graphs of the
sampler are cached per shape, the allocator reuses its blocks, and batches of jobs can share a length.
Bucket spacing is denser at small N so that the quadratic pair cost wasted on padding stays below ~1.56x.
"""

from __future__ import annotations

import dataclasses

import torch
import torch.nn.functional as F

BUCKET_SIZES = [128, 160, 192, 224, 256, 320, 384, 448, 512, 640, 768, 896, 1024, 1280, 1536, 1792, 2048, 2560, 3072,
                3584, 4096]  # fmt: skip
NOT_TOKEN_AXES = {"template_mask": (), "msa": (1,), "msa_mask": (1,), "deletion_matrix": (1,), "has_deletion": (1,),
                  "deletion_value": (1,)}  # fmt: skip


def bucket_size(n: int, buckets=BUCKET_SIZES) -> int:
    for b in buckets:
        if n <= b:
            return b
    return -(-n // 512) * 512


def _token_axes(key: str, t: torch.Tensor, n: int) -> tuple[int, ...]:
    if key in NOT_TOKEN_AXES:
        return tuple(a for a in NOT_TOKEN_AXES[key] if t.dim() > a and t.shape[a] == n)
    if key.startswith("template_"):
        return tuple(a for a in range(1, t.dim()) if t.shape[a] == n)[:2]
    return tuple(a for a in range(min(t.dim(), 2)) if t.shape[a] == n)


def pad_features(features: dict, n_pad: int | None = None) -> tuple[dict, int]:
    """Right-pad every token axis to ``n_pad`` (default: the bucket of the current length) with masked tokens.

    Returns the padded features and the original token count.
    """
    n = int(features["res_type"].shape[0])
    n_pad = bucket_size(n) if n_pad is None else n_pad
    if n_pad <= n:
        return features, n
    out = {}
    for k, v in features.items():
        if not isinstance(v, torch.Tensor) or v.dim() == 0:
            out[k] = v
            continue
        t = v
        for axis in _token_axes(k, v, n):
            pad = [0, 0] * (t.dim() - axis - 1) + [0, n_pad - n]
            t = F.pad(t, pad)
        out[k] = t
    return out, n


TOKEN_AXES_OF_OUTPUT = {"atom_positions": (1,), "atom_mask": (1,), "plddt": (1,), "pae": (1, 2), "pde": (1, 2),
                        "exp_resolved": (1,), "distogram": (0, 1)}  # fmt: skip


def unpad_output(output, n: int):
    """Cut every token axis of a ``DeepFold3Output`` back to ``n`` tokens."""
    fields = {}
    for f in dataclasses.fields(output):
        t = getattr(output, f.name)
        if isinstance(t, torch.Tensor):
            for axis in TOKEN_AXES_OF_OUTPUT.get(f.name, ()):
                if t.shape[axis] > n:
                    t = t.narrow(axis, 0, n)
        fields[f.name] = t
    return dataclasses.replace(output, **fields)
