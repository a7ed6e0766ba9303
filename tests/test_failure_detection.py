"""Failure handling exercised on the host with gloo ranks: no GPU is faulted, trapped or hung."""

import os
import subprocess
import sys

import pytest
import torch

from deepfold3_dev_b200.config.schema import TrainingConfig
from deepfold3_dev_b200.parallel.dist import DistInfo
from deepfold3_dev_b200.training.engine import OptimizerEngine
from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW
from deepfold3_dev_b200.training.scheduler import build_scheduler
from deepfold3_dev_b200.training.state import TrainState

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist_worker.py")


def _spawn(scenario, out_dir, port, world=2):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), PYTHONPATH=ROOT)
    return [subprocess.Popen([sys.executable, WORKER, scenario, str(out_dir)],
                             env=dict(env, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r))) for r in range(world)]  # fmt: skip


@pytest.mark.slow
def test_nan_on_one_rank_skips_on_all(tmp_path):
    assert [p.wait(timeout=600) for p in _spawn("nan_consensus", tmp_path, 29621)] == [0, 0]


def test_stop_file_reaches_every_rank(tmp_path):
    assert [p.wait(timeout=120) for p in _spawn("stop_file", tmp_path, 29622)] == [0, 0]


def test_missing_peer_surfaces_as_named_error(tmp_path):
    codes = [p.wait(timeout=120) for p in _spawn("peer_exits", tmp_path, 29623)]
    assert codes == [0, 0]


def _engine(limit):
    torch.manual_seed(0)
    model = torch.nn.Linear(4, 4)
    cfg = TrainingConfig(max_consecutive_nan_skips=limit, warmup_steps=0)
    opt = FlatAdamW(model, lr=1e-2)
    return model, opt, OptimizerEngine(opt, build_scheduler(opt, cfg), DistInfo(), cfg)


def test_nan_loss_skips_and_aborts_after_limit():
    model, opt, eng = _engine(limit=2)
    st = TrainState()
    before = opt.flat_param.clone()
    eng.add_microstep_loss(torch.tensor(float("nan")))
    res = eng.step_or_skip(st)
    assert not res.advanced and res.reason == "loss" and torch.equal(before, opt.flat_param)
    eng.add_microstep_loss(torch.tensor(float("inf")))
    with pytest.raises(RuntimeError, match="consecutive non-finite"):
        eng.step_or_skip(st)


def test_nan_gradient_skips_without_touching_parameters():
    model, opt, eng = _engine(limit=0)
    st = TrainState()
    model(torch.randn(2, 4)).sum().backward()
    opt.flat_grad[0] = float("nan")
    before = opt.flat_param.clone()
    eng.add_microstep_loss(torch.tensor(1.0))
    res = eng.step_or_skip(st)
    assert not res.advanced and res.reason == "grad" and torch.equal(before, opt.flat_param)
    assert float(opt.flat_grad.abs().sum()) == 0.0 and st.effective_step == 0
    model(torch.randn(2, 4)).sum().backward()
    eng.add_microstep_loss(torch.tensor(1.0))
    assert eng.step_or_skip(st).advanced and st.consecutive_nan_skips == 0


def test_gradient_outlier_threshold():
    model, opt, eng = _engine(limit=0)
    eng.cfg.grad_norm_skip_threshold = 1e-6
    model(torch.randn(2, 4)).sum().backward()
    eng.add_microstep_loss(torch.tensor(1.0))
    assert eng.step_or_skip(TrainState()).reason == "grad"
