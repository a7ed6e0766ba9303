"""Loader and Python face of the sm_100a extension (``ops/csrc``).

The extension is built in-tree by ``ops/build.py`` into
``ops/_df3_sm100.so`` and loaded with ``torch.ops.load_library``. On a box
with a GPU a missing or unloadable extension is an error; there is no silent
CPU or eager substitute for CUDA tensors.
"""

from __future__ import annotations

import os
import threading

import torch

_LOCK = threading.Lock()
_STATE: dict = {"loaded": False, "error": None, "features": frozenset()}
SO_NAME = "_df3_sm100.so"


def so_path() -> str:
    """The extension to load: the debug variant with index checks when ``DF3_BOUNDS_CHECK=1`` (built by
    ``python -m deepfold3_dev_b200.ops.build --checked``), else the normal one."""
    name = "_df3_sm100_checked.so" if os.environ.get("DF3_BOUNDS_CHECK", "0") == "1" else SO_NAME
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), name)


def _load() -> None:
    with _LOCK:
        if _STATE["loaded"] or _STATE["error"] is not None:
            return
        path = so_path()
        try:
            if not os.path.exists(path):
                raise FileNotFoundError(f"{path} not built; run `python -m deepfold3_dev_b200.ops.build`")
            torch.ops.load_library(path)
            feats = torch.ops.df3.features()
            _STATE["features"] = frozenset(feats.split(","))
            _STATE["loaded"] = True
        except Exception as exc:  # noqa: BLE001 - reported to the caller of require()
            _STATE["error"] = exc


class _Native:
    """Thin namespace over ``torch.ops.df3`` plus the autograd wrappers."""

    def has(self, feature: str) -> bool:
        if os.environ.get("DF3_DISABLE_OPS") and feature in os.environ["DF3_DISABLE_OPS"].split(","):
            return False
        return feature in _STATE["features"]

    def __getattr__(self, name):
        from . import autograd_ops

        return getattr(autograd_ops, name)


_NATIVE = _Native()


def available() -> bool:
    _load()
    return _STATE["loaded"]


def require() -> _Native:
    """The native namespace; raises if the extension cannot be loaded."""
    _load()
    if not _STATE["loaded"]:
        raise RuntimeError(
            "deepfold3_dev_b200: the sm_100a extension is required for CUDA tensors but failed to load: "
            f"{_STATE['error']!r}"
        )
    return _NATIVE
