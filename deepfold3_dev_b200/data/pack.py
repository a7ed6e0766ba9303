"""Pack shards: many small files in a few tar archives with an index (reference: data/pack.py:146-447).

A pack is a directory with ``shard-*.tar`` files and ``index.json`` (``{name: [shard, offset, size]}``).
``Pack.exists`` / ``Pack.read_bytes`` give random access through cached file descriptors and advise the
kernel to drop the pages afterwards, so a long run does not fill the page cache with training data.
"""

from __future__ import annotations

import json
import os
import tarfile
import threading


def build_pack(src_dir: str, out_dir: str, shard_bytes: int = 1 << 30) -> int:
    """Pack every file under ``src_dir`` (flat) into tar shards; returns the number of files."""
    os.makedirs(out_dir, exist_ok=True)
    index, shard, size, tar = {}, -1, shard_bytes, None
    for name in sorted(os.listdir(src_dir)):
        path = os.path.join(src_dir, name)
        if not os.path.isfile(path):
            continue
        if size >= shard_bytes:
            if tar is not None:
                tar.close()
            shard, size = shard + 1, 0
            tar = tarfile.open(os.path.join(out_dir, f"shard-{shard:05d}.tar"), "w")
        info = tar.gettarinfo(path, arcname=name)
        with open(path, "rb") as f:
            tar.addfile(info, f)
        index[name] = [shard, tar.offset - ((info.size + 511) // 512) * 512, info.size]
        size += info.size
    if tar is not None:
        tar.close()
    with open(os.path.join(out_dir, "index.json"), "w") as f:
        json.dump(index, f)
    return len(index)


class Pack:
    def __init__(self, root: str, max_open: int = 64):
        self.root = root
        with open(os.path.join(root, "index.json")) as f:
            self.index = json.load(f)
        self._fds: dict[int, int] = {}
        self._lock = threading.Lock()
        self.max_open = max_open

    def exists(self, name: str) -> bool:
        return name in self.index

    def _fd(self, shard: int) -> int:
        with self._lock:
            fd = self._fds.get(shard)
            if fd is None:
                if len(self._fds) >= self.max_open:
                    _, old = self._fds.popitem()
                    os.close(old)
                fd = os.open(os.path.join(self.root, f"shard-{shard:05d}.tar"), os.O_RDONLY)
                self._fds[shard] = fd
            return fd

    def read_bytes(self, name: str) -> bytes:
        shard, offset, size = self.index[name]
        fd = self._fd(shard)
        data = os.pread(fd, size, offset)
        if hasattr(os, "posix_fadvise"):
            os.posix_fadvise(fd, offset, size, os.POSIX_FADV_DONTNEED)
        return data

    def close(self) -> None:
        with self._lock:
            for fd in self._fds.values():
                os.close(fd)
            self._fds.clear()
