"""AlphaFold 3 parameter files (reference: params.py:13-87, convert/af3.py:274-913).

``read_af3_params`` parses the record stream of ``af3.bin`` / ``af3.bin.zst`` without JAX: each record is
five little-endian int32 (scope length, name length, dtype length, rank, payload bytes) followed by the
scope, the name, the dtype string, the shape and the raw array; bfloat16 is widened to float32.

``haiku_to_torch`` turns the nested ``{scope: {name: array}}`` into this package's state dict and
``torch_to_haiku`` goes back. Both are driven by one table (``convert/af3_name_map.py``): which Haiku scope
is which module, what kind of arrays it holds (a linear layer stored input-major or output-major, a layer
norm, a bare gain, ...) and how many leading axes are layer stacks. Compressed files need the
``zstandard`` package.
"""

from __future__ import annotations

import struct
import sys

import numpy as np
import torch

HEADER = struct.Struct("<5i")


def _read_record(stream):
    head = stream.read(HEADER.size)
    if not head:
        return None
    if len(head) < HEADER.size:
        raise ValueError("truncated record header")
    scope_len, name_len, dtype_len, rank, nbytes = HEADER.unpack(head)
    meta = struct.Struct(f"<{scope_len}s{name_len}s{dtype_len}s{rank}i")
    body = stream.read(meta.size + nbytes)
    if len(body) < meta.size + nbytes:
        raise ValueError("truncated record payload")
    scope, name, dtype, *shape = meta.unpack_from(body)
    raw = body[meta.size :]
    dtype = dtype.decode()
    if dtype == "bfloat16":
        arr = np.frombuffer(raw, dtype=np.uint16).reshape(shape)
        if sys.byteorder == "big":
            arr = arr.byteswap()
        arr = (arr.astype(np.uint32) << 16).view(np.float32)
    else:
        arr = np.frombuffer(raw, dtype=dtype).reshape(shape)
        if sys.byteorder == "big":
            arr = arr.byteswap()
    return scope.decode(), name.decode(), arr


def read_af3_params(path: str) -> dict[str, dict[str, np.ndarray]]:
    params: dict[str, dict[str, np.ndarray]] = {}
    with open(path, "rb") as f:
        stream = f
        if str(path).endswith(".zst"):
            try:
                import zstandard
            except ImportError as exc:
                raise RuntimeError("reading .zst parameter files needs the zstandard package; decompress the file first") from exc
            stream = zstandard.ZstdDecompressor().stream_reader(f)
        while (rec := _read_record(stream)) is not None:
            scope, name, arr = rec
            params.setdefault(scope, {})[name] = arr
    if not params:
        raise FileNotFoundError(f"no parameters found in {path}")
    return params


def haiku_to_torch(params: dict) -> dict[str, torch.Tensor]:
    """State dict from AF3's ``{scope: {name: array}}``; scopes the table does not know are reported with a warning."""
    from .af3_name_map import haiku_to_torch as convert

    return convert(params)


def torch_to_haiku(state_dict: dict) -> dict:
    """The inverse: AF3-layout ``{scope: {name: array}}`` (layers re-stacked) from a state dict of this model."""
    from .af3_name_map import torch_to_haiku as convert

    return convert(state_dict)


def convert_file(path: str, name_map: str | None = None) -> dict[str, torch.Tensor]:
    """``af3.bin`` / ``af3.bin.zst`` -> state dict. ``name_map`` is accepted for older call sites and ignored: the table
    ships with the package."""
    return haiku_to_torch(read_af3_params(path))
