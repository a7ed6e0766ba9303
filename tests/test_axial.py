"""Axial sharding of the pair tensor: push patterns against the collective statement, and the sharded Pairformer block
against the unsharded one (2 gloo ranks on CPU)."""

import os
import subprocess
import sys

import pytest
import torch

from deepfold3_dev_b200.parallel import peer_exchange as px

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4])
def test_push_patterns_state_the_relayouts(world):
    """The strided push plans, executed on the host for all ranks, give the re-layouts they are named for."""
    g = torch.Generator().manual_seed(0)
    B, n, C, G = 2, 3, 8, 2
    N = n * world
    z = torch.randn(B, N, N, C, generator=g)
    shards = [z[:, p * n : (p + 1) * n].contiguous() for p in range(world)]
    # transpose: rank q ends with rows q of z^T
    got = px.emulate([px.plan_transpose(tuple(s.shape), p, world) for p, s in enumerate(shards)], shards)
    zt = z.transpose(1, 2)
    for q in range(world):
        torch.testing.assert_close(got[q], zt[:, q * n : (q + 1) * n], atol=0, rtol=0)
    # all-gather along the row axis and along an inner axis
    for dim in (1, 2):
        parts = [torch.randn(B, 3, 5, generator=g) for _ in range(world)]
        got = px.emulate([px.plan_all_gather(tuple(t.shape), dim, p, world) for p, t in enumerate(parts)], parts)
        for q in range(world):
            torch.testing.assert_close(got[q], torch.cat(parts, dim), atol=0, rtol=0)
    # rows -> channels and back
    planes = torch.randn(G, C, B, N, N, generator=g)  # [group, channel, batch, row, column]
    by_rows = [planes[:, :, :, p * n : (p + 1) * n].contiguous() for p in range(world)]
    got = px.emulate([px.plan_rows_to_channels(tuple(t.shape), p, world) for p, t in enumerate(by_rows)], by_rows)
    cp = C // world
    for q in range(world):
        torch.testing.assert_close(got[q], planes[:, q * cp : (q + 1) * cp], atol=0, rtol=0)
    by_channels = [planes[0, q * cp : (q + 1) * cp].contiguous() for q in range(world)]
    got = px.emulate([px.plan_channels_to_rows(tuple(t.shape), p, world) for p, t in enumerate(by_channels)], by_channels)
    for q in range(world):
        torch.testing.assert_close(got[q], planes[0][:, :, q * n : (q + 1) * n], atol=0, rtol=0)


def test_plans_reject_shapes_that_do_not_split():
    with pytest.raises(ValueError):
        px.plan_transpose((1, 3, 10, 8), 0, 4)
    with pytest.raises(ValueError):
        px.plan_rows_to_channels((2, 6, 1, 2, 8), 0, 4)
    with pytest.raises(ValueError):
        px.plan_channels_to_rows((2, 1, 9, 9), 0, 2)


@pytest.mark.slow
@pytest.mark.parametrize("world", [2, 4])
def test_sharded_pairformer_equals_unsharded_on_gloo(tmp_path, world):
    script = os.path.join(ROOT, "tests", "dist_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(29640 + world), PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, script, "axial_block", str(tmp_path)],
                              env=dict(env, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r))) for r in range(world)]  # fmt: skip
    for p in procs:
        assert p.wait(timeout=600) == 0
    for r in range(world):
        res = torch.load(tmp_path / f"axial_rank{r}.pt")
        assert float(res["scale"]) > 0.1
        assert float(res["pair_err"]) < 2e-5 * max(1.0, float(res["scale"])), res
        assert float(res["single_err"]) < 2e-5 and float(res["msa_err"]) < 2e-5, res
