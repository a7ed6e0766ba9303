"""Packs: a directory tree of many small files stored as a few tar shards plus a sorted index.

File systems with a file-count quota cannot hold tens of millions of small feature files. A pack keeps the original
bytes of every file as a member of an uncompressed tar shard (``tar tf`` still lists them) and records where each
member's data starts, so a read is one binary search and one ``pread``.

On-disk layout, the one the reference writes (data/pack.py:1-60), so packs interchange::

    {root}/_pack/meta.json        {"format": "deepfold3-pack", "version": 1, "files": n, "shards": k, "include": [...]}
    {root}/_pack/keys.npy         sorted fixed-width byte strings: paths relative to {root}, '/' separated
    {root}/_pack/loc.npy          per key (shard <u4, offset <u8, size <u8)
    {root}/_pack/SHA256SUMS       one line per shard
    {root}/_pack/shards/00000.tar ...

A pack directory written by earlier versions of this package (``index.json`` + ``shard-00000.tar``) is still read.

Path transparency: loaders keep asking for ordinary paths. ``register(root)`` (called by the datasets on
construction) notes that ``{root}/_pack`` exists; afterwards ``lookup(path)`` answers for any path below a registered
root, and ``data.io_cache.read_bytes`` / ``exists`` go through it. Whether the pack is authoritative for a path (a
miss means "no such file", without a ``stat``) is decided by ``include`` prefixes when the pack has them, else by the
first path component: a whole-tree pack covers every top-level name that occurs among its keys, so small files left
beside ``_pack/`` (``manifest.json``) still come from the file system. Registered roots are mirrored into
``DEEPFOLD3_PACK_ROOTS`` for spawned worker processes; descriptors are reopened after a fork.

The builder is resumable: shards are written one at a time under a temporary name, a state file lists the finished
ones with their members, and a rerun continues after the last finished shard.
"""

from __future__ import annotations

import hashlib
import json
import os
import tarfile
import threading
from collections import OrderedDict

import numpy as np

PACK_DIRNAME = "_pack"
FORMAT = "deepfold3-pack"
VERSION = 1
ENV_ROOTS = "DEEPFOLD3_PACK_ROOTS"
ENV_MAX_FDS = "DEEPFOLD3_PACK_MAX_FDS"
LOC_DTYPE = np.dtype([("shard", "<u4"), ("offset", "<u8"), ("size", "<u8")])
_BLOCK = 512


# ------------------------------------------------------------------------------------------------------------ building
def _walk(src_dir: str, include: tuple[str, ...]):
    """Relative '/'-separated paths of the regular files under ``src_dir`` (sorted), skipping any ``_pack`` directory."""
    out = []
    for base, dirs, files in os.walk(src_dir, followlinks=True):
        dirs[:] = sorted(d for d in dirs if d != PACK_DIRNAME)
        rel = os.path.relpath(base, src_dir)
        for name in files:
            key = name if rel == "." else f"{rel}/{name}".replace(os.sep, "/")
            if not include or key.startswith(include):
                out.append(key)
    out.sort()
    return out


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while chunk := f.read(1 << 24):
            h.update(chunk)
    return h.hexdigest()


def build_pack(src_dir: str, out_dir: str, shard_bytes: int = 1 << 30, include=()) -> int:
    """Pack the files under ``src_dir`` (recursively; only those under the ``include`` prefixes when given) into
    ``out_dir``; returns the number of files. Safe to rerun after an interruption."""
    include = tuple(include)
    shards_dir = os.path.join(out_dir, "shards")
    state_path = os.path.join(out_dir, "_build", "state.json")
    os.makedirs(shards_dir, exist_ok=True)
    os.makedirs(os.path.dirname(state_path), exist_ok=True)
    state = {"shards": []}  # per finished shard: [[key, offset, size], ...]
    if os.path.exists(state_path):
        with open(state_path) as f:
            state = json.load(f)
    keys = _walk(src_dir, include)
    done = {k for members in state["shards"] for k, _, _ in members}
    todo = [k for k in keys if k not in done]

    def flush(tar, tmp, members):
        tar.close()
        os.replace(tmp, os.path.join(shards_dir, f"{len(state['shards']):05d}.tar"))
        state["shards"].append(members)
        with open(state_path + ".tmp", "w") as f:
            json.dump(state, f)
        os.replace(state_path + ".tmp", state_path)

    tar, tmp, members, size = None, None, [], 0
    for key in todo:
        if tar is None:
            tmp = os.path.join(shards_dir, f".{len(state['shards']):05d}.tar.part")
            tar, members, size = tarfile.open(tmp, "w", format=tarfile.GNU_FORMAT), [], 0
        path = os.path.join(src_dir, key)
        info = tar.gettarinfo(path, arcname=key)
        if not info.isreg():  # a link to a file: store the file
            info = tar.gettarinfo(os.path.realpath(path), arcname=key)
        with open(path, "rb") as f:
            tar.addfile(info, f)
        padded = (info.size + _BLOCK - 1) // _BLOCK * _BLOCK
        members.append([key, tar.offset - padded, info.size])
        size += info.size
        if size >= shard_bytes:
            flush(tar, tmp, members)
            tar = None
    if tar is not None:
        flush(tar, tmp, members)

    rows = [(k, s, off, n) for s, ms in enumerate(state["shards"]) for k, off, n in ms]
    rows.sort()
    width = max((len(k.encode()) for k, *_ in rows), default=1)
    key_arr = np.array([k.encode() for k, *_ in rows], dtype=f"S{width}")
    loc = np.zeros(len(rows), dtype=LOC_DTYPE)
    loc["shard"], loc["offset"], loc["size"] = ([r[i] for r in rows] for i in (1, 2, 3))
    np.save(os.path.join(out_dir, "keys.npy"), key_arr)
    np.save(os.path.join(out_dir, "loc.npy"), loc)
    with open(os.path.join(out_dir, "SHA256SUMS"), "w") as f:
        for s in range(len(state["shards"])):
            f.write(f"{_sha256(os.path.join(shards_dir, f'{s:05d}.tar'))}  shards/{s:05d}.tar\n")
    meta = {"format": FORMAT, "version": VERSION, "files": len(rows), "shards": len(state["shards"]),
            "bytes": int(loc["size"].sum()), "include": list(include)}  # fmt: skip
    with open(os.path.join(out_dir, "meta.json.tmp"), "w") as f:
        json.dump(meta, f, indent=1)
    os.replace(os.path.join(out_dir, "meta.json.tmp"), os.path.join(out_dir, "meta.json"))
    return len(rows)


# ------------------------------------------------------------------------------------------------------------- reading
def _max_fds() -> int:
    """Open shard descriptors kept per process: a quarter of the soft limit, at most 1024. A worker that runs for days
    touches every shard, and an unbounded cache ends in EMFILE, which loaders would report as unreadable records."""
    if os.environ.get(ENV_MAX_FDS):
        return max(1, int(os.environ[ENV_MAX_FDS]))
    try:
        import resource

        soft = resource.getrlimit(resource.RLIMIT_NOFILE)[0]
        soft = 1 << 20 if soft == resource.RLIM_INFINITY else soft
    except (ImportError, OSError, ValueError):
        soft = 1024
    return max(16, min(1024, soft // 4))


class _Descriptors:
    """Process-wide least-recently-used table of open shard files; forgotten (not closed) in a forked child."""

    def __init__(self):
        self.pid, self.table, self.lock = None, OrderedDict(), threading.Lock()

    def get(self, path: str) -> int:
        with self.lock:
            if self.pid != os.getpid():
                self.pid, self.table, self.limit = os.getpid(), OrderedDict(), _max_fds()
            fd = self.table.get(path)
            if fd is not None:
                self.table.move_to_end(path)
                return fd
            fd = os.open(path, os.O_RDONLY)
            if hasattr(os, "posix_fadvise"):
                try:
                    os.posix_fadvise(fd, 0, 0, os.POSIX_FADV_RANDOM)  # single members at random: no read-ahead
                except OSError:
                    pass
            self.table[path] = fd
            while len(self.table) > self.limit:
                _, old = self.table.popitem(last=False)
                os.close(old)
            return fd

    def forget(self, prefix: str) -> None:
        with self.lock:
            for path in [p for p in self.table if p.startswith(prefix)]:
                os.close(self.table.pop(path))


_FDS = _Descriptors()


class Pack:
    """Random access to one pack directory: ``exists(key)``, ``read_bytes(key)``, ``keys()``, ``covers(key)``."""

    def __init__(self, root: str, max_open: int | None = None):
        self.root = str(root)
        self.legacy = not os.path.exists(os.path.join(self.root, "meta.json"))
        if self.legacy:
            with open(os.path.join(self.root, "index.json")) as f:
                self.index = json.load(f)
            self.meta, self.include = {"files": len(self.index)}, ()
        else:
            with open(os.path.join(self.root, "meta.json")) as f:
                self.meta = json.load(f)
            if self.meta.get("format") != FORMAT:
                raise ValueError(f"{self.root}: not a {FORMAT} directory (format={self.meta.get('format')!r})")
            if int(self.meta.get("version", 0)) > VERSION:
                raise ValueError(f"{self.root}: pack version {self.meta['version']} is newer than {VERSION}")
            self.include = tuple(self.meta.get("include") or ())
        self._pid = self._keys = self._loc = self._tops = None
        self._lock = threading.Lock()

    def _open(self):
        if self._pid != os.getpid():
            with self._lock:
                if self._pid != os.getpid():
                    if not self.legacy:  # memory-mapped: shared through the page cache by all workers of a node
                        self._keys = np.load(os.path.join(self.root, "keys.npy"), mmap_mode="r")
                        self._loc = np.load(os.path.join(self.root, "loc.npy"), mmap_mode="r")
                    self._pid = os.getpid()

    def __len__(self) -> int:
        return int(self.meta["files"])

    def keys(self) -> list[str]:
        if self.legacy:
            return sorted(self.index)
        self._open()
        return [k.decode() for k in self._keys]

    def _find(self, key: str):
        if self.legacy:
            hit = self.index.get(key)
            return None if hit is None else (f"shard-{hit[0]:05d}.tar", hit[1], hit[2])
        self._open()
        raw = key.encode()
        if not raw or len(raw) > self._keys.dtype.itemsize:
            return None
        i = int(np.searchsorted(self._keys, np.array(raw, dtype=self._keys.dtype)))
        if i >= len(self._keys) or self._keys[i] != raw:
            return None
        row = self._loc[i]
        return f"shards/{int(row['shard']):05d}.tar", int(row["offset"]), int(row["size"])

    def exists(self, key: str) -> bool:
        return self._find(key) is not None

    def covers(self, key: str) -> bool:
        """Is this pack the authority for ``key`` (so that a miss means the file does not exist)?"""
        if self.include:
            return key.startswith(self.include) or (key + "/").startswith(self.include)
        if self._tops is None:
            self._tops = {k.split("/", 1)[0] for k in self.keys()}
        return key.split("/", 1)[0] in self._tops

    def is_dir(self, key: str) -> bool:
        prefix = key.rstrip("/") + "/"
        if self.legacy:
            return any(k.startswith(prefix) for k in self.index)
        self._open()
        i = int(np.searchsorted(self._keys, np.array(prefix.encode()[: self._keys.dtype.itemsize], dtype=self._keys.dtype)))
        return i < len(self._keys) and bytes(self._keys[i]).startswith(prefix.encode())

    def read_bytes(self, key: str) -> bytes:
        hit = self._find(key)
        if hit is None:
            raise FileNotFoundError(f"{key!r} is not in the pack {self.root}")
        shard, offset, size = hit
        fd = _FDS.get(os.path.join(self.root, shard))
        data = os.pread(fd, size, offset)
        if len(data) != size:
            raise OSError(f"short read of {key!r} from {self.root}/{shard}: {len(data)} of {size} bytes (truncated shard?)")
        from . import io_cache

        if io_cache.dropping() and hasattr(os, "posix_fadvise"):
            try:
                os.posix_fadvise(fd, offset, size, os.POSIX_FADV_DONTNEED)
            except OSError:
                pass
        return data

    def close(self) -> None:
        _FDS.forget(self.root)


# ------------------------------------------------------------------------------------------------------ path transparency
_ROOTS: dict[str, Pack] = {}
_ENV_SEEN = ""


def register(root: str) -> Pack | None:
    """Note the pack of a dataset root (``{root}/_pack``), if there is one; returns its reader."""
    root = os.path.abspath(str(root))
    if root in _ROOTS:
        return _ROOTS[root]
    pack_dir = os.path.join(root, PACK_DIRNAME)
    if not (os.path.exists(os.path.join(pack_dir, "meta.json")) or os.path.exists(os.path.join(pack_dir, "index.json"))):
        return None
    _ROOTS[root] = Pack(pack_dir)
    known = [r for r in os.environ.get(ENV_ROOTS, "").split(os.pathsep) if r]
    if root not in known:
        os.environ[ENV_ROOTS] = os.pathsep.join(known + [root])
    return _ROOTS[root]


def unregister_all() -> None:
    for p in _ROOTS.values():
        p.close()
    _ROOTS.clear()
    os.environ.pop(ENV_ROOTS, None)


def _sync_env() -> None:
    global _ENV_SEEN
    env = os.environ.get(ENV_ROOTS, "")
    if env != _ENV_SEEN:  # a spawned worker starts with the variable but an empty table
        _ENV_SEEN = env
        for root in env.split(os.pathsep):
            if root and root not in _ROOTS:
                register(root)


def lookup(path: str):
    """``(pack, key, state)`` for a path: state ``"hit"`` (in the pack), ``"miss"`` (the pack is the authority for this
    part of the tree and does not have it) or ``"pass"`` (no pack says anything: ask the file system)."""
    _sync_env()
    if not _ROOTS:
        return None, None, "pass"
    full = os.path.abspath(str(path))
    for root, pk in _ROOTS.items():
        if full.startswith(root + os.sep):
            key = full[len(root) + 1 :].replace(os.sep, "/")
            if pk.exists(key):
                return pk, key, "hit"
            return pk, key, "miss" if pk.covers(key) else "pass"
    return None, None, "pass"
