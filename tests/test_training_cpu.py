"""Training runtime on CPU: flat optimizer vs torch.optim.AdamW, schedules, checkpoint round trip, gloo DDP step."""

import copy
import os
import subprocess
import sys

import pytest
import torch

from deepfold3_dev_b200.config.schema import TrainingConfig
from deepfold3_dev_b200.data.synthetic import batch_features, synthetic_complex
from deepfold3_dev_b200.models.model import DeepFold3
from deepfold3_dev_b200.parallel.dist import DistInfo
from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW
from deepfold3_dev_b200.training.scheduler import build_scheduler
from deepfold3_dev_b200.training.trainer import Trainer
from tests.helpers import tiny_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mlp():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(7, 13), torch.nn.LayerNorm(13), torch.nn.Linear(13, 3))


def test_flat_adamw_matches_torch_adamw_and_ema():
    a, b = _mlp(), _mlp()
    ref = torch.optim.AdamW(a.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    shadow = [p.detach().clone() for p in a.parameters()]
    opt = FlatAdamW(b, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, ema_decay=0.9)
    x = torch.randn(5, 7)
    for _ in range(4):
        for m in (a, b):
            m(x).pow(2).sum().backward()
        ref.step()
        ref.zero_grad()
        torch._foreach_lerp_(shadow, [p.detach() for p in a.parameters()], 0.1)
        opt.step()
        opt.zero_grad()
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(q, p, atol=1e-6, rtol=1e-5)
    ema = opt.ema_state_dict()["shadow"]
    for (n, _), s in zip(b.named_parameters(), shadow):
        torch.testing.assert_close(ema[n], s, atol=1e-6, rtol=1e-5)


def test_flat_adamw_state_dict_roundtrip_is_torch_layout():
    a = _mlp()
    opt = FlatAdamW(a, lr=1e-2, ema_decay=0.5)
    a(torch.randn(2, 7)).sum().backward()
    opt.step()
    sd = opt.state_dict()
    assert set(sd) == {"state", "param_groups"} and set(sd["state"][0]) == {"step", "exp_avg", "exp_avg_sq"}
    b = _mlp()
    opt2 = FlatAdamW(b, lr=1e-2, ema_decay=0.5)
    opt2.load_state_dict(copy.deepcopy(sd))
    torch.testing.assert_close(opt2.exp_avg, opt.exp_avg)
    assert opt2.step_count == 1
    # torch's own AdamW accepts the same dict
    c = _mlp()
    groups = [{"params": [p for n, p in c.named_parameters() if p.dim() >= 2]},
              {"params": [p for n, p in c.named_parameters() if p.dim() < 2]}]  # fmt: skip
    torch.optim.AdamW(groups, lr=1e-2).load_state_dict(sd)


def test_no_decay_rules():
    from deepfold3_dev_b200.training.flat_optimizer import is_no_decay

    assert is_no_decay("x.norm.weight", torch.zeros(8))
    assert is_no_decay("a.to_g.weight", torch.zeros(8, 8))
    assert is_no_decay("evoformer.bond_embedding.weight", torch.zeros(8, 1))
    assert not is_no_decay("a.to_q.weight", torch.zeros(8, 8))


def test_schedulers():
    cfg = TrainingConfig(warmup_steps=10, start_decay_after=20, decay_every=5, decay_factor=0.5, lr=1.0)
    opt = FlatAdamW(_mlp(), lr=1.0)
    s = build_scheduler(opt, cfg)
    lrs = []
    for _ in range(31):
        lrs.append(s.get_last_lr()[0])
        s.step()
    assert lrs[0] == 0.0 and abs(lrs[5] - 0.5) < 1e-9 and lrs[10] == 1.0 and lrs[19] == 1.0
    assert lrs[20] == 1.0 and lrs[25] == 0.5 and lrs[30] == 0.25
    cfg2 = TrainingConfig(warmup_steps=2, finetune_scheduler="cosine", finetune_max_steps=12, finetune_min_lr_ratio=0.1, lr=1.0)
    s2 = build_scheduler(FlatAdamW(_mlp(), lr=1.0), cfg2)
    assert abs(s2.multiplier(12) - 0.1) < 1e-9 and s2.multiplier(2) == 1.0
    cfg3 = TrainingConfig(warmup_steps=0, finetune_scheduler="wsds", wsds_decay_windows=[[10, 20]], wsds_min_lr_ratio=0.1, lr=1.0)
    s3 = build_scheduler(FlatAdamW(_mlp(), lr=1.0), cfg3)
    assert s3.multiplier(5) == 1.0 and s3.multiplier(10) == 1.0 and s3.multiplier(20) == 1.0 and s3.multiplier(19) < 0.2


@pytest.mark.slow
def test_trainer_step_checkpoint_resume(tmp_path):
    mc = tiny_config()
    tc = TrainingConfig(diffusion_batch_size=2, dtype="fp32", mini_rollout_steps=2, max_recycles=1, warmup_steps=2,
                        output_dir=str(tmp_path), seed=3)  # fmt: skip
    batch = batch_features([synthetic_complex([("protein", 12), ("protein", 8)], num_msa=8, num_templates=1, seed=1)])
    tr = Trainer(tc, mc, dist_info=DistInfo())
    out = [tr.train_step(copy.deepcopy(batch), num_recycles=1) for _ in range(2)]
    assert all(o["advanced"] for o in out) and tr.state.effective_step == 2
    path = tr.save_checkpoint(background=False)
    blob = torch.load(path, weights_only=False)
    for key in ("model", "optimizer", "optimizer_param_names", "scheduler", "global_step", "effective_step", "epoch",
                "best_eval_loss", "rng_states", "model_cfg", "train_cfg", "snapshot_kind", "ema", "scaler", "sampler"):  # fmt: skip
        assert key in blob, key
    assert set(blob["ema"]) == {"decay", "num_updates", "shadow"}
    after = tr.train_step(copy.deepcopy(batch), num_recycles=1)
    tr2 = Trainer(tc, mc, dist_info=DistInfo())
    tr2.load_checkpoint(path)
    assert tr2.state.effective_step == 2
    again = tr2.train_step(copy.deepcopy(batch), num_recycles=1)
    assert abs(again["loss"] - after["loss"]) < 1e-5 * max(1.0, abs(after["loss"]))
    assert abs(again["grad_norm"] - after["grad_norm"]) < 1e-4 * max(1.0, after["grad_norm"])


@pytest.mark.slow
def test_gloo_two_ranks_match_single_process(tmp_path):
    """World size 2 over gloo: averaged gradients equal the single-process gradient of the two-example batch mean."""
    script = os.path.join(ROOT, "tests", "dist_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, script, "ddp_step", str(tmp_path)],
                              env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r))) for r in range(2)]  # fmt: skip
    for p in procs:
        assert p.wait(timeout=600) == 0
    a, b = (torch.load(tmp_path / f"rank{r}.pt") for r in range(2))
    torch.testing.assert_close(a["params"], b["params"])  # ranks stay in lock step
    single = subprocess.run([sys.executable, script, "single_step", str(tmp_path)], env=env, timeout=600)
    assert single.returncode == 0
    ref = torch.load(tmp_path / "single.pt")
    torch.testing.assert_close(a["grad"], ref["grad"], atol=2e-5, rtol=1e-3)


@pytest.mark.slow
def test_schedule_free_ranks_stay_in_lock_step(tmp_path):
    script = os.path.join(ROOT, "tests", "dist_worker.py")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", PYTHONPATH=ROOT)
    procs = [subprocess.Popen([sys.executable, script, "schedule_free_lockstep", str(tmp_path)],
                              env=dict(env, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r))) for r in range(2)]  # fmt: skip
    for p in procs:
        assert p.wait(timeout=600) == 0
    a, b = (torch.load(tmp_path / f"sf_rank{r}.pt") for r in range(2))
    torch.testing.assert_close(a["params"], b["params"], atol=0, rtol=0)
    torch.testing.assert_close(a["z"], b["z"], atol=0, rtol=0)


def test_schedule_free_checkpoint_follows_reference_layout(tmp_path):
    """Saved under eval mode: ``model`` = x, snapshot_kind "x", train_mode False; loading returns to y and can step."""
    from deepfold3_dev_b200.training.checkpointing import CheckpointManager
    from deepfold3_dev_b200.training.schedule_free import FlatAdamWScheduleFree
    from deepfold3_dev_b200.training.state import TrainState

    def make():
        m = _mlp()
        return m, FlatAdamWScheduleFree(m, lr=1e-2, warmup_steps=2)

    m, opt = make()
    x = torch.randn(5, 7)
    for _ in range(3):
        m(x).pow(2).sum().backward()
        opt.step()
        opt.zero_grad()
    y_before, z_before = opt.flat_param.clone(), opt.z.clone()
    b1 = opt.param_groups[0]["betas"][0]
    x_iter = torch.lerp(y_before, z_before, 1.0 - 1.0 / b1)
    sched = build_scheduler(opt, TrainingConfig(lr=1e-2))
    mgr = CheckpointManager(str(tmp_path), DistInfo())
    path = mgr.save("checkpoint_3.pt", model=m, optimizer=opt, scheduler=sched, state=TrainState(), model_cfg=None,
                    train_cfg=None, background=False)  # fmt: skip
    torch.testing.assert_close(opt.flat_param, y_before)  # back in train mode after the save
    blob = torch.load(path, weights_only=False)
    assert blob["snapshot_kind"] == "x" and blob["optimizer"]["param_groups"][0]["train_mode"] is False
    saved = torch.cat([blob["model"][n].reshape(-1) for n, _ in m.named_parameters()])
    live_x = torch.cat([opt._view(x_iter, i).reshape(-1) for i in range(len(opt.params))])
    torch.testing.assert_close(saved, live_x)
    m2, opt2 = make()
    mgr.load(path, model=m2, optimizer=opt2, scheduler=build_scheduler(opt2, TrainingConfig(lr=1e-2)), state=TrainState())
    assert opt2.train_mode
    torch.testing.assert_close(opt2.flat_param, y_before, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(opt2.z, z_before)
    m2(x).pow(2).sum().backward()
    opt2.step()  # does not raise
    mgr.close()


@pytest.mark.slow
def test_hourly_checkpoint_timer_restarts_after_each_save(tmp_path):
    """With the wall-clock trigger due at once, exactly one checkpoint is written per elapsed period, not one per step."""
    from deepfold3_dev_b200.data.datasets import SyntheticDataset

    mc = tiny_config()
    tc = TrainingConfig(diffusion_batch_size=2, dtype="fp32", mini_rollout_steps=1, max_recycles=0, warmup_steps=0,
                        output_dir=str(tmp_path), seed=3, max_steps=3, checkpoint_interval=1000, checkpoint_every_hours=1.0,
                        log_interval=100, alpha_confidence=0.0)  # fmt: skip
    batch = batch_features([synthetic_complex([("protein", 10)], num_msa=4, num_templates=0, seed=1)])
    tr = Trainer(tc, mc, dist_info=DistInfo(), train_loader=[batch, batch, batch, batch])
    saved = []
    real = tr.save_checkpoint
    tr.save_checkpoint = lambda name=None, background=True: (saved.append(name), real(name, background))[1]
    import time as _time

    tr_run_time = _time.time
    # first optimizer step sees a timer that ran out long ago; later ones see a fresh timer
    orig_after = tr._after_optimizer_step

    def after(req):
        if tr.state.effective_step == 1:
            tr._last_ckpt_wall = tr_run_time() - 7200
        return orig_after(req)

    tr._after_optimizer_step = after
    tr.run()
    periodic = [n for n in saved if n is None]
    assert len(periodic) == 1, saved
