"""Model-level checks on the GPU: the native path agrees with the CPU fp32 path, and a training step runs."""

import copy

import pytest
import torch

from deepfold3_dev_b200 import ops
from deepfold3_dev_b200.config.schema import TrainingConfig
from deepfold3_dev_b200.data.synthetic import batch_features, synthetic_complex
from deepfold3_dev_b200.models.model import DeepFold3
from deepfold3_dev_b200.parallel.dist import DistInfo
from deepfold3_dev_b200.training.trainer import Trainer
from tests.helpers import tiny_config, wake_zero_init

pytestmark = pytest.mark.gpu


def test_trunk_distogram_gpu_fp32_matches_cpu():
    torch.manual_seed(0)
    cfg = tiny_config()
    cpu = DeepFold3(cfg).eval()
    wake_zero_init(cpu)
    gpu = copy.deepcopy(cpu).cuda()
    feats = synthetic_complex([("protein", 40), ("protein", 24)], num_msa=12, num_templates=1, seed=4, with_gt=False)
    with torch.no_grad():
        a = cpu.compute_distogram(copy.deepcopy(feats), num_recycles=1)
        b = gpu.compute_distogram({k: v.cuda() for k, v in feats.items()}, num_recycles=1)
    torch.testing.assert_close(b.cpu(), a, atol=5e-3, rtol=5e-3)
    assert any(k.endswith(":sm100") for k in ops.census())


def test_bf16_training_step_runs_and_updates():
    mc = tiny_config()
    tc = TrainingConfig(diffusion_batch_size=4, dtype="bf16", mini_rollout_steps=2, max_recycles=1, warmup_steps=0,
                        alpha_pae=1.0, output_dir="/tmp/df3_test_gpu")  # fmt: skip
    tr = Trainer(tc, mc, dist_info=DistInfo(device=torch.device("cuda", 0)))
    batch = batch_features([synthetic_complex([("protein", 48), ("protein", 32)], num_msa=16, num_templates=2, seed=1)])
    before = tr.optimizer.flat_param.clone()
    outs = [tr.train_step(copy.deepcopy(batch), num_recycles=1) for _ in range(2)]
    assert all(o["advanced"] and o["loss"] == o["loss"] for o in outs)
    assert not torch.equal(before, tr.optimizer.flat_param)
    assert tr.optimizer.ema_updates == 2
