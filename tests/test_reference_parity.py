"""Same weights, same features, same seed: this model against the reference package, on CPU in fp32."""

import copy

import pytest
import torch

from deepfold3_dev_b200.config import schema as MC
from deepfold3_dev_b200.data.synthetic import batch_features, synthetic_complex
from deepfold3_dev_b200.models.model import DeepFold3
from tests.helpers import small_full_width, wake_zero_init


@pytest.fixture(scope="module")
def pair(reference_package):
    import deepfold3.model.config as RC
    from deepfold3.model.model import DeepFold3 as RefModel

    torch.manual_seed(0)
    ref = RefModel(small_full_width(RC))
    wake_zero_init(ref)
    mine = DeepFold3(small_full_width(MC))
    mine.load_state_dict(ref.state_dict(), strict=True)
    return ref, mine


def test_state_dict_layout_matches(reference_package):
    import deepfold3.model.config as RC
    from deepfold3.model.model import DeepFold3 as RefModel

    ref = {k: tuple(v.shape) for k, v in RefModel(small_full_width(RC)).state_dict().items()}
    mine = {k: tuple(v.shape) for k, v in DeepFold3(small_full_width(MC)).state_dict().items()}
    assert ref == mine


def test_config_fields_match(reference_package):
    import dataclasses

    import deepfold3.model.config as RC

    for name in ("ModelConfig", "TrainingConfig", "OptimConfig", "PrecisionConfig", "DiffusionConfig", "DataConfig",
                 "EvoformerConfig", "PairFormerConfig", "ConfidenceConfig", "TemplateEmbeddingConfig",
                 "DatasetConfig", "DistogramConfig", "MaskedMSAConfig"):  # fmt: skip
        a = {f.name: repr(getattr(getattr(RC, name)(), f.name)) for f in dataclasses.fields(getattr(RC, name))}
        b = {f.name: repr(getattr(getattr(MC, name)(), f.name)) for f in dataclasses.fields(getattr(MC, name))}
        assert a == b, name


def test_inference_forward_matches(pair):
    ref, mine = pair
    ref.eval()
    mine.eval()
    feats = synthetic_complex([("protein", 8), ("protein", 6), ("ligand", 3)], num_msa=6, num_templates=2, seed=2,
                              with_gt=False)  # fmt: skip
    with torch.no_grad():
        a = ref(copy.deepcopy(feats), seed=3)
        b = mine(copy.deepcopy(feats), seed=3)
    for key in ("distogram", "plddt", "pae", "pde", "exp_resolved"):
        torch.testing.assert_close(getattr(b, key), getattr(a, key), atol=2e-4, rtol=1e-4)
    scale = a.atom_positions.abs().max()
    assert (a.atom_positions - b.atom_positions).abs().max() < 1e-5 * scale


@pytest.mark.parametrize("chunk", [0, 2])
def test_training_loss_and_gradients_match(pair, chunk):
    import deepfold3.model.config as RC
    from deepfold3.training.collectives import slice_batch_dict
    from deepfold3.training.loss import training_loss as ref_loss

    from deepfold3_dev_b200.training.objective import training_loss

    ref, mine = pair
    ref.train()
    mine.train()
    feats = batch_features([synthetic_complex([("protein", 8), ("protein", 7, "x"), ("protein", 7, "x"), ("ligand", 3)],
                                              num_msa=6, num_templates=2, seed=1)])  # fmt: skip

    def run(model, loss_fn, cfg):
        torch.manual_seed(5)
        model.zero_grad()
        f = copy.deepcopy(feats)
        pred = model.forward_training(
            f, num_recycles=1, diffusion_batch_size=4, mini_rollout_steps=2, seed=0, diffusion_chunk_size=chunk,
            backward_fn=(lambda l: l.backward()) if chunk else None, loss_cfg=cfg if chunk else None,
            permute_gt_before_noise=True,
        )  # fmt: skip
        loss, parts = loss_fn(slice_batch_dict(pred, 0, 1), slice_batch_dict(f, 0, 1), cfg)
        loss.backward()
        grads = torch.cat([(p.grad if p.grad is not None else torch.zeros_like(p)).reshape(-1) for p in model.parameters()])
        return loss.detach(), {k: float(v) for k, v in parts.items()}, grads

    la, pa, ga = run(ref, ref_loss, RC.TrainingConfig(alpha_pae=1.0, diffusion_chunk_size=chunk))
    lb, pb, gb = run(mine, training_loss, MC.TrainingConfig(alpha_pae=1.0, diffusion_chunk_size=chunk))
    assert abs(float(la) - float(lb)) < 1e-4 * max(1.0, abs(float(la)))
    for k, v in pa.items():
        assert abs(v - pb[k]) < 1e-4 * max(1.0, abs(v)), k
    assert (ga - gb).abs().max() < 1e-4 * ga.abs().max()


@pytest.mark.parametrize("head_norm,router,kind", [("channel", True, "softmax"), ("head_rms", False, "softmax"), ("head_rms", True, "sigmoid"),
                                                   ("head_ln", True, "softmax"), ("post_channel", True, "softmax")])  # fmt: skip
def test_multi_head_triangle_multiply_matches(reference_package, head_norm, router, kind):
    """Per-head normalisation and routing of the triangle multiply against the reference module, router statistics included."""
    import deepfold3.model.ops as RO

    from deepfold3_dev_b200.models import triangle as T

    torch.manual_seed(1)
    kw = dict(num_heads=4, head_norm=head_norm, router=router, router_kind=kind)
    ref = RO.TriangleMulOutgoing(32, **kw)
    wake_zero_init(ref)
    mine = T.TriangleMulOutgoing(32, **kw)
    mine.load_state_dict(ref.state_dict(), strict=True)
    z, mask = torch.randn(1, 9, 9, 32), (torch.rand(1, 9, 9) > 0.2).float()
    if router:
        RO.set_router_stats_enabled(ref, True)
        T.set_router_stats_enabled(mine, True)
    torch.testing.assert_close(mine(z, mask), ref(z, mask), atol=1e-5, rtol=1e-4)
    if router:
        a, b = RO.collect_router_stats(ref), T.collect_router_stats(mine)
        assert a.keys() == b.keys()
        for k in a:
            assert abs(a[k] - b[k]) < 1e-5 * max(1.0, abs(a[k])), k
