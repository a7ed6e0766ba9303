"""Complex language model: scopes of the layer kinds, muP groups, store round trip, masking, packing, a short training run."""

import json
import os

import numpy as np
import pytest
import torch

from deepfold3_dev_b200.complexlm.config import ComplexLMConfig, DataConfig, ExperimentConfig, MaskingConfig, SourceConfig, TrainConfig, load_experiment
from deepfold3_dev_b200.complexlm.data import (ComplexStore, ComplexStoreWriter, Example, SourceView, apply_masking, crop_complex,
                                               eligible_indices, pack)  # fmt: skip
from deepfold3_dev_b200.complexlm.model import IGNORE_INDEX, MASK_ID, ComplexLM, decode, encode, swiglu_hidden
from deepfold3_dev_b200.complexlm.prepare import cluster_stores, store_stats
from deepfold3_dev_b200.complexlm.trainer import ComplexLMTrainer, lr_at

A = "MKTAYIAKQRQISFVKSHFSRQLEERLGLIEVQ"
B = "GSHMSEQNNTEMTFQIQRIYTKDISFEAPNAPHVFQ"


def _example(seqs, entity, source=0):
    toks = [encode(s).astype(np.int64) for s in seqs]
    labels = [np.where(np.arange(len(t)) % 5 == 0, t, IGNORE_INDEX) for t in toks]
    return Example(toks, labels, [0] * len(seqs), np.asarray(entity), [np.zeros(len(t), bool) for t in toks], False, source)


def _small(**kw):
    return ComplexLMConfig(d_model=64, n_heads=4, n_layers=4, attn_impl="sdpa", **kw)


def test_vocab_roundtrip():
    assert decode(encode("ACDXZ")) == "ACDXZ" and int(encode("L")[0]) == 4


def test_layer_scopes():
    torch.manual_seed(0)
    batch = pack([_example([A, B], [0, 1]), _example([A], [0], 1)])
    assert batch.n_chains == 3 and batch.n_complexes == 2 and batch.n_tokens == 2 * len(A) + len(B)
    assert int(batch.positions[len(A)]) == 0 and int(batch.global_positions[len(A)]) == len(A)

    def changed(pattern):
        m = ComplexLM(_small(layer_pattern=pattern)).eval()
        with torch.no_grad():
            base = m(batch).logits
            alt_tokens = batch.tokens.clone()
            alt_tokens[len(A) + 3] = 7  # edit chain B of complex 0
            alt = pack([_example([A, B], [0, 1]), _example([A], [0], 1)])
            alt.tokens = alt_tokens
            diff = (m(alt).logits - base).abs().amax(-1)
        a, b, c = diff[: len(A)].max(), diff[len(A) : len(A) + len(B)].max(), diff[len(A) + len(B) :].max()
        return float(a), float(b), float(c)

    a, b, c = changed("c")
    assert a == 0 and b > 0 and c == 0  # chain-scoped: only chain B moves
    a, b, c = changed("cg")
    assert a > 0 and b > 0 and c == 0  # complex-scoped layers carry it to chain A, never to the other complex
    a, b, c = changed("x")
    assert a > 0 and c == 0


def test_homomer_equals_monomer_under_global_layers():
    torch.manual_seed(0)
    m = ComplexLM(_small(layer_pattern="cg")).eval()
    with torch.no_grad():
        mono = m(pack([_example([A], [0])])).logits
        homo = m(pack([_example([A, A, A], [0, 0, 0])])).logits
    assert torch.allclose(homo[: len(A)], mono, atol=1e-5) and torch.allclose(homo[len(A) : 2 * len(A)], mono, atol=1e-5)


def test_mup_groups_and_names():
    cfg = ComplexLMConfig(d_model=128, n_heads=4, n_layers=2, attn_impl="sdpa", mup=True, mup_base_width=64)
    m = ComplexLM(cfg)
    groups = {g["role"]: g for g in m.param_groups(0.01) if g["weight_decay"] > 0}
    assert groups["hidden"]["lr_scale"] == pytest.approx(0.5) and groups["hidden"]["weight_decay"] == pytest.approx(0.02)
    assert groups["readout"]["lr_scale"] == 1.0 and m.readout_mult == pytest.approx(0.5)
    keys = set(m.state_dict())
    assert {"embed.weight", "blocks.0.attn.qkv.weight", "blocks.0.attn.q_norm.weight", "blocks.1.ffn.w_in.weight",
            "blocks.1.ffn.w_out.weight", "norm.weight", "head.dense.weight", "head.out.bias"} <= keys  # fmt: skip
    assert swiglu_hidden(1280, 8 / 3) == 3584
    with pytest.raises(ValueError):
        ComplexLMConfig(layer_pattern="cx", attn_impl="varlen")


def _write_store(root, n=24, with_iface=True):
    rng = np.random.default_rng(0)
    w = ComplexStoreWriter(root, "toy", with_iface)
    letters = np.array(list("ACDEFGHIKLMNPQRSTVWY"))
    for i in range(n):
        a = "".join(rng.choice(letters, 40))
        b = "".join(rng.choice(letters, 30))
        seqs = [a, a] if i % 3 == 0 else ([a, b] if i % 3 == 1 else [a])
        iface = [rng.random(len(s)) < 0.2 for s in seqs] if with_iface else None
        w.add(f"cx{i}", seqs, iface, date=20200101 + i if i % 4 else 0)
    return w.close()


def test_store_roundtrip_and_views(tmp_path):
    root = str(tmp_path / "toy")
    info = _write_store(root)
    assert info["complexes"] == 24
    s = ComplexStore(root)
    cx = s.example(0)
    assert cx.is_homomer and len(cx.chains) == 2 and cx.entity[0] == cx.entity[1] and cx.iface[0].dtype == bool
    assert not s.example(1).is_homomer
    st = store_stats(root)
    assert st["homomers"] == 8 and st["heteromers"] == 8 and st["monomers"] == 8
    undated_dropped = eligible_indices(s, SourceConfig(name="toy", date_max=20200110))
    assert all(int(s.cx_date[i]) > 0 and int(s.cx_date[i]) <= 20200110 for i in undated_dropped)
    held = eligible_indices(s, SourceConfig(name="toy", holdout_every=4, holdout_side="eval"))
    assert list(held) == [0, 4, 8, 12, 16, 20]
    res = cluster_stores([root])
    assert res["complex_clusters"] >= 1 and ComplexStore(root).meta["cluster_run"] == res["cluster_run"]
    view = SourceView(ComplexStore(root), SourceConfig(name="toy"), DataConfig(data_root=str(tmp_path)))
    rng = np.random.default_rng(0)
    assert all(0 <= view.draw(rng) < 24 for _ in range(20))


def test_masking_and_crop():
    rng = np.random.default_rng(0)
    ids = encode(A * 20).astype(np.int64)
    toks, labels = apply_masking(rng, [ids, ids], np.array([0, 0]), None, MaskingConfig(), False)
    assert np.array_equal(toks[0], toks[1]) and np.array_equal(labels[0], labels[1])  # copies share one draw
    sel = labels[0] != IGNORE_INDEX
    assert 0.10 < sel.mean() < 0.20 and 0.7 < (toks[0][sel] == MASK_ID).mean() < 0.9
    assert np.array_equal(toks[0][~sel], ids[~sel])
    t2, l2 = apply_masking(rng, [ids, ids], np.array([0, 0]), None, MaskingConfig(homomer_paired=False), False)
    assert not np.array_equal(l2[0], l2[1])
    flags = np.zeros(len(ids), bool)
    flags[:200] = True
    _, l3 = apply_masking(rng, [ids], np.array([0]), [flags], MaskingConfig(), True)
    assert (l3[0][:200] != IGNORE_INDEX).mean() > (l3[0][200:] != IGNORE_INDEX).mean() + 0.05
    wins = crop_complex(rng, [300, 300, 100], np.array([0, 0, 1]), None, max_chain_len=120, max_complex_len=350)
    assert wins[0] == wins[1] and wins[0][1] - wins[0][0] <= 120 and sum(b - a for a, b in wins) <= 350


def test_config_overrides(tmp_path):
    (tmp_path / "base.yaml").write_text("model:\n  d_model: 128\n  n_heads: 4\ntrain:\n  lr: 0.001\n")
    (tmp_path / "child.yaml").write_text("base: base.yaml\nmodel:\n  n_layers: 2\ndata:\n  sources:\n    - name: toy\n      weight: 2.0\n")
    cfg = load_experiment(str(tmp_path / "child.yaml"), {"model.layer_pattern": "ccg", "train.max_steps": "7"})
    assert cfg.model.d_model == 128 and cfg.model.n_layers == 2 and cfg.model.kinds == ["c", "c"]
    assert cfg.train.max_steps == 7 and cfg.data.sources[0].weight == 2.0 and cfg.train.lr == 0.001
    assert lr_at(0, cfg.train) < lr_at(cfg.train.warmup_steps, cfg.train)


def test_short_training_run_learns(tmp_path):
    _write_store(str(tmp_path / "toy"), n=12)
    cfg = ExperimentConfig(
        model=_small(layer_pattern="cg"),
        data=DataConfig(data_root=str(tmp_path), sources=[SourceConfig(name="toy")], token_budget=600, num_workers=0),
        train=TrainConfig(max_steps=40, lr=3e-3, warmup_steps=4, log_every=0, eval_every=0, save_every=0, dtype="fp32"),
        eval_sources=[SourceConfig(name="toy", interface_masking=True)],
    )
    tr = ComplexLMTrainer(cfg, str(tmp_path / "run"), device="cpu")
    it = iter(tr.stream)
    first = tr.train_step([next(it)])
    for _ in range(39):
        last = tr.train_step([next(it)])
    assert last["loss"] < first["loss"] - 0.3  # 12 fixed complexes are memorised quickly
    ev = tr.evaluate()
    assert "all/loss" in ev and "all/delta" in ev and abs(ev.get("homomer/delta", 0.0)) < 1e-3
    path = tr.save_checkpoint(final=True)
    tr2 = ComplexLMTrainer(cfg, str(tmp_path / "run2"), resume=path, device="cpu")
    assert tr2.step == 40 and json.load(open(os.path.join(tmp_path, "run", "config.json")))["model"]["d_model"] == 64


def test_esmc_warm_start_copies_every_tensor(tmp_path):
    """A stand-in ESM-C checkpoint (its parameter names, a 64-row token table) loads tensor for tensor: names translate,
    the vocabulary axis takes the leading rows, nothing is left random; misfits and missing tensors are errors."""
    from deepfold3_dev_b200.complexlm import esmc
    from deepfold3_dev_b200.complexlm.config import load_experiment

    cfg = _small(norm="layernorm", esmc_compat=True, mup=False)
    model = ComplexLM(cfg)
    inverse = {}
    for name, p in model.named_parameters():
        module, _, leaf = name.rpartition(".")
        src = {"embed": "embed", "norm": "transformer.norm", "head.dense": "sequence_head.0", "head.norm": "sequence_head.2",
               "head.out": "sequence_head.3"}.get(module)  # fmt: skip
        if src is None:
            i, rest = module.split(".")[1], ".".join(module.split(".")[2:])
            src = f"transformer.blocks.{i}." + {"attn.norm": "attn.layernorm_qkv.0", "attn.qkv": "attn.layernorm_qkv.1", "attn.q_norm": "attn.q_ln",
                                                 "attn.k_norm": "attn.k_ln", "attn.out_proj": "attn.out_proj", "ffn.norm": "ffn.0",
                                                 "ffn.w_in": "ffn.1", "ffn.w_out": "ffn.3"}[rest]  # fmt: skip
        inverse[f"{src}.{leaf}"] = name
    assert all(esmc.translate(k) == v for k, v in inverse.items()) and esmc.translate("transformer.blocks.0.attn.rotary.inv_freq") is None
    torch.manual_seed(1)
    state = {}
    for src, name in inverse.items():
        p = dict(model.named_parameters())[name]
        shape = (64, *p.shape[1:]) if name in ("embed.weight", "head.out.weight", "head.out.bias") else p.shape
        state[src] = torch.randn(*shape)
    state["transformer.blocks.0.attn.rotary.inv_freq"] = torch.ones(4)
    path = tmp_path / "esmc.pth"
    torch.save({"state_dict": state}, path)
    report = esmc.load_esmc(model, str(path))
    assert report["copied"] == len(inverse) and report["left_random"] == [] and report["unused_source"] == ["transformer.blocks.0.attn.rotary.inv_freq"]
    got = dict(model.named_parameters())
    assert torch.equal(got["embed.weight"], state["embed.weight"][:33]) and torch.equal(got["head.out.bias"], state["sequence_head.3.bias"][:33])
    assert torch.equal(got["blocks.1.ffn.w_in.weight"], state["transformer.blocks.1.ffn.1.weight"])
    del state["transformer.norm.weight"]
    torch.save(state, path)
    with pytest.raises(ValueError, match="got nothing"):
        esmc.load_esmc(model, str(path))
    assert esmc.load_esmc(model, str(path), strict=False)["left_random"] == ["norm.weight"]
    state["transformer.blocks.0.ffn.1.weight"] = torch.zeros(3, 3)
    torch.save(state, path)
    with pytest.raises(ValueError, match="does not fit"):
        esmc.load_esmc(model, str(path), strict=False)
    with pytest.raises(ValueError, match="esmc_compat"):
        esmc.load_esmc(ComplexLM(_small()), str(path))
    big = load_experiment(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "configs", "plm-esmc600m.yaml"))
    assert esmc.matching_release(big.model) == "esmc-600m" and big.model.esmc_compat and not big.model.mup and big.train.lr == 1.0e-4


def test_diagnostics_permutation_and_sinks():
    from deepfold3_dev_b200.complexlm.diagnostics import attention_sink_stats, permutation_sensitivity

    torch.manual_seed(0)
    ex = _example([A, B], [0, 1])
    inv = permutation_sensitivity(ComplexLM(_small(layer_pattern="cg")), ex, [1, 0])
    assert abs(inv["loss_change"]) < 1e-4 and inv["token_cosine_min"] > 0.9999  # chain order is invisible to this pattern
    dep = permutation_sensitivity(ComplexLM(_small(layer_pattern="r")), ex, [1, 0])
    assert dep["token_cosine_min"] < 0.9999  # rotary positions over the concatenation see the order
    stats = attention_sink_stats(ComplexLM(_small(layer_pattern="cg")), pack([ex]))
    assert [s["kind"] for s in stats] == ["c", "g", "c", "g"] and all(s["x_uniform"] >= 1.0 for s in stats)


@pytest.mark.gpu
def test_packed_segment_attention_matches_dense_on_gpu():
    """The variable-length path (CUDA, bf16) and the dense masked path give the same logits."""
    torch.manual_seed(0)
    batch = pack([_example([A, B], [0, 1]), _example([A, A], [0, 0], 1)]).to("cuda")
    cfg_v = ComplexLMConfig(d_model=64, n_heads=4, n_layers=4, layer_pattern="cg", attn_impl="varlen")
    model = ComplexLM(cfg_v).cuda().bfloat16().eval()
    with torch.no_grad():
        packed = model(batch).logits.float()
        for blk in model.blocks:
            blk.attn.cfg = ComplexLMConfig(d_model=64, n_heads=4, n_layers=4, layer_pattern="cg", attn_impl="sdpa")
        dense = model(batch).logits.float()
    assert (packed - dense).abs().max() < 0.05 * dense.abs().max() + 1e-2
