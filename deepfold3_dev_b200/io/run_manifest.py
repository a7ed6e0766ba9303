"""``run_manifest.json``: what ran, on what, with which inputs (reference: io/run_manifest.py:26-112)."""

from __future__ import annotations

import hashlib
import json
import os
import platform
import subprocess
import sys
import time


def _run(*cmd: str) -> str | None:
    try:
        return subprocess.run(cmd, capture_output=True, text=True, timeout=10, check=True).stdout.strip()
    except Exception:  # noqa: BLE001
        return None


def git_state() -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    return {"commit": _run("git", "-C", here, "rev-parse", "HEAD"), "dirty": bool(_run("git", "-C", here, "status", "--porcelain"))}


def runtime_versions() -> dict:
    import torch

    return {"python": sys.version.split()[0], "torch": torch.__version__, "cuda": torch.version.cuda,
            "platform": platform.platform()}  # fmt: skip


def gpu_name(device) -> str | None:
    import torch

    return torch.cuda.get_device_name(device) if torch.cuda.is_available() and str(device).startswith("cuda") else None


def sha256_file(path: str, chunk_size: int = 1 << 24) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while chunk := f.read(chunk_size):
            h.update(chunk)
    return h.hexdigest()


def checkpoint_record(path: str) -> dict:
    return {"path": os.path.abspath(path), "bytes": os.path.getsize(path), "sha256": sha256_file(path)}


def new_manifest(**fields) -> dict:
    return {"status": "running", "started": time.strftime("%Y-%m-%dT%H:%M:%S"), "argv": sys.argv, "git": git_state(),
            "versions": runtime_versions(), **fields}  # fmt: skip


def write_manifest(path: str, manifest: dict) -> None:
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(manifest, f, indent=1, default=str)
    os.replace(tmp, path)
