"""Reads that do not pollute the page cache (reference: data/io_cache.py:43-99).

A training run streams terabytes of small files once each; left alone they evict everything useful from the page
cache. With dropping enabled every file is advised out of the cache right after it was read.
"""

from __future__ import annotations

import io
import os

import numpy as np

_DROP = False


def set_drop_page_cache(enabled: bool) -> None:
    global _DROP
    _DROP = bool(enabled)


def dropping() -> bool:
    return _DROP


def drop_from_page_cache(fd: int) -> None:
    if _DROP and hasattr(os, "posix_fadvise"):
        try:
            os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_DONTNEED)
        except OSError:
            pass


def read_bytes(path: str) -> bytes:
    """The bytes of a file, taken from the pack of a registered dataset root when the file lives there."""
    from . import pack

    pk, key, state = pack.lookup(path)
    if state == "hit":
        return pk.read_bytes(key)
    if state == "miss":
        raise FileNotFoundError(f"{path}: not in the pack that covers this part of {pk.root}")
    with open(path, "rb") as f:
        data = f.read()
        drop_from_page_cache(f.fileno())
    return data


def exists(path: str) -> bool:
    """``os.path.exists`` that asks the pack first (no ``stat`` for paths a pack is the authority for)."""
    from . import pack

    pk, key, state = pack.lookup(path)
    if state == "pass":
        return os.path.exists(path)
    return state == "hit" or pk.is_dir(key)


def read_text(path: str, encoding: str = "utf-8") -> str:
    return read_bytes(path).decode(encoding)


def read_npz(path: str, allow_pickle: bool = False):
    """The arrays of an ``.npz`` file as a dict, read through one buffered pass."""
    with np.load(io.BytesIO(read_bytes(path)), allow_pickle=allow_pickle) as z:
        return {k: z[k] for k in z.files}
