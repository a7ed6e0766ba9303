"""AlphaFold 3 parameter files (reference: params.py:13-87, convert/af3.py:274-913).

``read_af3_params`` parses the record stream of ``af3.bin`` / ``af3.bin.zst`` without JAX: each record is
five little-endian int32 (scope length, name length, dtype length, rank, payload bytes) followed by the
scope, the name, the dtype string, the shape and the raw array; bfloat16 is widened to float32.

``convert_file`` turns the nested ``{scope: {name: array}}`` into this package's state dict through a
name map: a JSON list of rules ``{"scope": regex, "name": regex, "key": template, "transpose": bool,
"stack_axis": int | null}``. Layer-stacked arrays (haiku ``layer_stack``) are split along ``stack_axis``
and ``{layer}`` in the template is replaced by the index; regex groups are available as ``{1}``, ``{2}``.
The map for the published AF3 checkpoint is data, not code; it is not bundled here because it cannot be
validated without the checkpoint. Compressed files need the ``zstandard`` package.
"""

from __future__ import annotations

import json
import re
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


def apply_name_map(params: dict, rules: list[dict]) -> dict[str, torch.Tensor]:
    compiled = [(re.compile(r["scope"]), re.compile(r.get("name", ".*")), r) for r in rules]
    out: dict[str, torch.Tensor] = {}
    unmatched = []
    for scope, entries in params.items():
        for name, arr in entries.items():
            for sre, nre, rule in compiled:
                ms, mn = sre.fullmatch(scope), nre.fullmatch(name)
                if not (ms and mn):
                    continue
                groups = (None,) + ms.groups() + mn.groups()  # "{1}" is the first regex group
                t = torch.from_numpy(np.array(arr, copy=True)).float()
                axis = rule.get("stack_axis")
                pieces = [(None, t)] if axis is None else list(enumerate(t.unbind(axis)))
                for layer, piece in pieces:
                    if rule.get("transpose"):
                        piece = piece.transpose(-1, -2)
                    key = rule["key"].format(*groups, layer=layer)
                    out[key] = piece.contiguous()
                break
            else:
                unmatched.append(f"{scope}/{name}")
    if unmatched:
        raise KeyError(f"{len(unmatched)} arrays match no rule of the name map (first: {unmatched[:5]})")
    return out


def convert_file(path: str, name_map: str | None = None) -> dict[str, torch.Tensor]:
    params = read_af3_params(path)
    if name_map is None:
        raise RuntimeError("AF3 conversion needs a name map (JSON rules from haiku scopes to state-dict keys): "
                           "convert_file(path, name_map='af3_name_map.json')")  # fmt: skip
    with open(name_map) as f:
        return apply_name_map(params, json.load(f))
