"""Model-level checks on the GPU: the native path agrees with the CPU fp32 path, and a training step runs."""

import copy
import os

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
    # the bf16 weight mirror follows the optimizer: the tensor-core path sees the updated parameters
    torch.testing.assert_close(tr.optimizer.flat_param_bf16.float(), tr.optimizer.flat_param.bfloat16().float())
    feats = {k: v[0].cuda() if torch.is_tensor(v) else v for k, v in batch.items()}
    outs = []
    for disable in ("", "gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,gemm"):
        os.environ["DF3_DISABLE_OPS"] = disable
        try:
            with torch.autocast("cuda", dtype=torch.bfloat16):
                outs.append(tr.model.compute_distogram(dict(feats), num_recycles=0).float())
        finally:
            os.environ.pop("DF3_DISABLE_OPS", None)
    assert ((outs[0] - outs[1]).norm() / outs[1].norm()).item() < 5e-2


def _block_grads(block, z, s, mask, disable):
    import os

    os.environ["DF3_DISABLE_OPS"] = disable
    try:
        for p in block.parameters():
            p.grad = None
        zz, ss = z.clone().requires_grad_(True), s.clone().requires_grad_(True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            zo, so = block(zz, ss, mask, mask[:, 0])
            loss = zo.float().square().mean() + so.float().square().mean()
        loss.backward()
        grads = {n: p.grad.clone() for n, p in block.named_parameters() if p.grad is not None}
        return zo.detach().float(), zz.grad.float(), grads
    finally:
        os.environ.pop("DF3_DISABLE_OPS", None)


def test_pairformer_block_fused_kernels_match_eager_bf16():
    """Forward and gradients of one Pairformer block: tensor-core kernels vs the eager bf16 statement."""
    from deepfold3_dev_b200.models.evoformer import PairFormerBlock

    torch.manual_seed(3)
    cfg = tiny_config()
    pf = cfg.pairformer
    block = PairFormerBlock(pf.pair_channel, pf.seq_channel, num_single_heads=pf.single_attention_num_head,
                            single_key_dim=pf.single_key_dim, single_value_dim=pf.single_value_dim, pair_dropout=0.0,
                            optim=cfg.optim).cuda().train()  # fmt: skip
    wake_zero_init(block)
    N = 136
    z = torch.randn(1, N, N, pf.pair_channel, device="cuda")
    s = torch.randn(1, N, pf.seq_channel, device="cuda")
    mask = torch.ones(1, N, N, device="cuda")
    mask[:, :, -5:] = 0
    mask[:, -5:, :] = 0
    fused_names = "gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,gemm"
    ops.census(reset=True)
    zo_f, dz_f, g_f = _block_grads(block, z, s, mask, "")
    assert ops.census().get("pair_bias_attention:sm100", 0) > 0
    zo_e, dz_e, g_e = _block_grads(block, z, s, mask, fused_names)

    def rel(a, b):
        return ((a - b).norm() / (b.norm() + 1e-12)).item()

    assert rel(zo_f - z, zo_e - z) < 3e-2
    assert rel(dz_f, dz_e) < 5e-2
    # gradients that are zero in exact arithmetic (a bias added before a softmax over the same axis) hold
    # only rounding noise in both runs, so each parameter is judged against the largest gradient as well
    top = max(g.float().norm().item() for g in g_e.values())
    for n in g_e:
        diff = (g_f[n].float() - g_e[n].float()).norm().item()
        assert diff <= 8e-2 * g_e[n].float().norm().item() + 2e-3 * top, (n, diff, g_e[n].float().norm().item())
    assert torch.ops.df3.gemm_status() == 0


@pytest.mark.parametrize("triangle_attention,single_track", [(False, False), (True, True)])
def test_wide_pair_block_fused_kernels_match_eager_bf16(triangle_attention, single_track):
    """The production recipe's block shape (pair width 256, 8 pair heads of 32; its stage-0 family also drops the
    triangle attention layers and the single track): kernels against the eager bf16 statement, forward and gradients."""
    from deepfold3_dev_b200.models.evoformer import PairFormerBlock

    torch.manual_seed(5)
    block = PairFormerBlock(256, 384, num_pair_heads=8, pair_dropout=0.0, use_triangle_attention=triangle_attention,
                            use_single_track=single_track).cuda().train()  # fmt: skip
    wake_zero_init(block)
    N = 72
    z = torch.randn(1, N, N, 256, device="cuda")
    s = torch.randn(1, N, 384, device="cuda")
    mask = torch.ones(1, N, N, device="cuda")
    mask[:, :, -3:] = 0
    mask[:, -3:, :] = 0
    fused_names = "gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,gemm"
    ops.census(reset=True)
    zo_f, dz_f, g_f = _block_grads(block, z, s, mask, "")
    seen = ops.census()
    assert any(k.startswith("triangle") and k.endswith(":sm100") and n > 0 for k, n in seen.items()), seen
    assert not any(k.startswith("triangle") and k.endswith(":torch") and n > 0 for k, n in seen.items()), seen
    assert (seen.get("pair_bias_attention:sm100", 0) > 0) == (triangle_attention or single_track)
    zo_e, dz_e, g_e = _block_grads(block, z, s, mask, fused_names)

    def rel(a, b):
        return ((a - b).norm() / (b.norm() + 1e-12)).item()

    assert rel(zo_f - z, zo_e - z) < 3e-2
    assert rel(dz_f, dz_e) < 5e-2
    top = max(g.float().norm().item() for g in g_e.values())
    for n in g_e:
        diff = (g_f[n].float() - g_e[n].float()).norm().item()
        assert diff <= 8e-2 * g_e[n].float().norm().item() + 2e-3 * top, (n, diff, g_e[n].float().norm().item())
    assert torch.ops.df3.gemm_status() == 0


def test_graphed_sampler_equals_eager_sampler(monkeypatch):
    """The CUDA-graph replay of the denoiser gives the sampler's eager result, also on a second (cached) call."""
    torch.manual_seed(1)
    cfg = tiny_config()
    cfg.diffusion.steps = 8
    cfg.diffusion.num_samples = 2
    model = DeepFold3(cfg).cuda().eval()
    wake_zero_init(model)
    feats = {k: v.cuda() for k, v in synthetic_complex([("protein", 30), ("protein", 20)], num_msa=8, num_templates=1,
                                                      seed=2, with_gt=False).items()}  # fmt: skip
    outs = {}
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        trunk = model.run_evoformer(feats, 0)
        for mode in ("0", "1", "1"):
            monkeypatch.setenv("DF3_GRAPH_SAMPLER", mode)
            outs.setdefault(mode, []).append(model.sample_from_trunk(feats, trunk, seed=5).atom_positions.float())
    graphs = model.diffusion_head.__dict__.get("_denoiser_graphs")
    assert graphs is not None and not graphs.failed and len(graphs._graphs) == 1
    eager, first, second = outs["0"][0], outs["1"][0], outs["1"][1]
    assert torch.isfinite(eager).all()
    torch.testing.assert_close(first, eager, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(second, first, atol=0, rtol=0)


def test_graphed_trunk_pass_equals_eager_and_redraws_dropout(monkeypatch):
    """No-grad trunk passes replayed from a CUDA graph: same result as eager in eval mode, fresh masks in train mode."""
    torch.manual_seed(2)
    cfg = tiny_config()
    model = DeepFold3(cfg).cuda()
    wake_zero_init(model)
    feats = {k: v.cuda() for k, v in synthetic_complex([("protein", 40), ("protein", 24)], num_msa=12, num_templates=1,
                                                      seed=4, with_gt=False).items()}  # fmt: skip

    def trunk(mode):
        monkeypatch.setenv("DF3_GRAPH_TRUNK", mode)
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            return model.run_evoformer(dict(feats), 1, seed=3)[0]["pair"].float()

    model.eval()
    eager, first, second = trunk("0"), trunk("1"), trunk("1")
    graphs = model.__dict__.get("_trunk_graphs")
    # two shape signatures: the first pass starts from fp32 zeros, later passes from the bf16 output of the previous one
    assert graphs is not None and not graphs.failed and 1 <= len(graphs._graphs) <= 2
    n_eval = len(graphs._graphs)
    torch.testing.assert_close(first, eager, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(second, first, atol=0, rtol=0)
    model.train()  # dropout on: replays must not repeat the mask
    a, b = trunk("1"), trunk("1")
    assert len(graphs._graphs) > n_eval  # the training flag is part of the cache key
    assert not torch.equal(a, b)
    assert torch.isfinite(a).all() and torch.isfinite(b).all()


def test_diffusion_transformer_fast_path_equals_block_by_block(monkeypatch):
    """The inference path with stacked conditioning products and epilogue-fused gates gives what the per-block
    statement gives (bf16 tolerance), with and without a sample axis on the conditioning."""
    from deepfold3_dev_b200.models.diffusion_modules import DiffusionTransformer
    from tests.helpers import wake_zero_init

    torch.manual_seed(0)
    net = DiffusionTransformer(256, 128, num_blocks=4, num_heads=8, super_block_size=2, c_pair=64).cuda().eval()
    wake_zero_init(net)
    B, S, N = 1, 3, 136
    act = torch.randn(B, S, N, 256, device="cuda")
    pair = torch.randn(B, N, N, 64, device="cuda")
    mask = torch.ones(B, N, device="cuda")
    mask[:, -3:] = 0
    for cond_samples in (1, S):
        cond = torch.randn(B, cond_samples, N, 128, device="cuda")
        with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
            logits = net.hoist_pair_logits(pair, mask)
            assert net._fast_ok(act, logits)
            fast = net.run(act, cond, logits)
            monkeypatch.setenv("DF3_DIFFUSION_FAST", "0")
            slow = net.run(act, cond, logits)
            monkeypatch.delenv("DF3_DIFFUSION_FAST")
        err = (fast.float() - slow.float()).pow(2).mean().sqrt() / slow.float().pow(2).mean().sqrt()
        assert float(err) < 1.5e-2, float(err)
