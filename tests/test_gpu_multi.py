"""Tests that need two or more GPUs: run as child processes, one per GPU, over NCCL with NVLS off."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(scenario: str, nproc: int, port: int) -> str:
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "gpu_dist_worker.py"), scenario]  # fmt: skip
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    return out.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_memory_gradient_reduction_matches_nccl():
    assert "WORKER_OK peer_reduce" in _run("peer_reduce", 2, 29631)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_optimizer_step_matches_nccl_and_torch_adamw():
    out = _run("fused_step", 2, 29633)
    assert "WORKER_OK fused_step" in out and out.count("FUSED_STEP ok") == 2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_axial_exchanges_match_collectives():
    assert "AXIAL_EXCHANGE ok" in _run("axial_exchange", 2, 29635)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_row_sharded_pairformer_matches_one_gpu():
    assert "AXIAL_BLOCK ok" in _run("axial_block", 2, 29637)
