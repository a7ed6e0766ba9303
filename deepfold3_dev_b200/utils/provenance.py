"""Who ran what: git state, command line, versions, GPU name (reference: scripts/train.py:48-106, io/run_manifest.py)."""

from __future__ import annotations

import os
import platform
import subprocess
import sys


def _git(*args: str) -> str:
    try:
        return subprocess.run(["git", *args], capture_output=True, text=True, timeout=5,
                              cwd=os.path.dirname(os.path.abspath(__file__))).stdout.strip()  # fmt: skip
    except Exception:  # noqa: BLE001
        return ""


def provenance() -> dict:
    import torch

    gpu = torch.cuda.get_device_name(0) if torch.cuda.is_available() else None
    return {
        "command": " ".join(sys.argv),
        "cwd": os.getcwd(),
        "git_commit": _git("rev-parse", "HEAD"),
        "git_dirty": bool(_git("status", "--porcelain")),
        "python": platform.python_version(),
        "torch": str(torch.__version__),
        "cuda": None if torch.version.cuda is None else str(torch.version.cuda),
        "gpu": gpu,
        "hostname": platform.node(),
    }
