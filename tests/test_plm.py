"""Language-model frontend: ESM-2 encoder against the transformers implementation, chain packing, pair projection."""

import pytest
import torch

from deepfold3_dev_b200.data import const
from deepfold3_dev_b200.models.plm import ESM2Config, ESM2Encoder, FrozenPLM, LMPairShim, esm2_tokenizer


def _small_cfg():
    return ESM2Config(hidden_size=64, num_hidden_layers=3, num_attention_heads=4, intermediate_size=128)


def test_encoder_matches_transformers(tmp_path):
    tr = pytest.importorskip("transformers")
    from safetensors.torch import save_file

    cfg = _small_cfg()
    hf_cfg = tr.EsmConfig(vocab_size=33, hidden_size=64, num_hidden_layers=3, num_attention_heads=4, intermediate_size=128,
                          position_embedding_type="rotary", token_dropout=True, emb_layer_norm_before=False, pad_token_id=1,
                          mask_token_id=32, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-5)  # fmt: skip
    torch.manual_seed(0)
    hf = tr.EsmModel(hf_cfg, add_pooling_layer=False).eval()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(tmp_path / "model.safetensors"))
    enc = ESM2Encoder(cfg).eval()
    enc.load_hf_safetensors(str(tmp_path / "model.safetensors"))
    ids = torch.tensor([[0, 5, 6, 7, 8, 9, 10, 2], [0, 11, 12, 32, 2, 1, 1, 1]])
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=(ids != 1).long(), output_hidden_states=True).hidden_states
        got = enc(ids)
    assert got.shape == (2, 8, 4, 64)
    real = ids != 1
    for layer in range(4):
        ref = want[layer] if layer < 3 else hf(input_ids=ids, attention_mask=(ids != 1).long()).last_hidden_state
        assert torch.allclose(got[:, :, layer][real], ref[real], atol=2e-5), layer


def test_tokenizer_table():
    tok = esm2_tokenizer()
    assert int(tok.res_type_to_id[const.RES_TYPE_ORDER["LEU"]]) == 4 and int(tok.res_type_to_id[const.RES_TYPE_ORDER["ALA"]]) == 5
    assert int(tok.res_type_to_id[const.RES_TYPE_ORDER["DA"]]) == tok.unk_id


def test_per_chain_equals_running_alone_and_scatter():
    torch.manual_seed(1)
    plm = FrozenPLM(cfg=_small_cfg(), join="per_chain")
    plm.load("cpu", torch.float32, random_init=True)
    # chain 0: 5 residues, the 3rd atomised into 3 atom tokens; chain 1: 4 residues; one ligand token
    res_type = torch.tensor([0, 1, 2, 2, 2, 3, 4, 5, 6, 7, 8, 20])
    asym = torch.tensor([0, 0, 0, 0, 0, 0, 0, 1, 1, 1, 1, 2])
    resid = torch.tensor([1, 2, 3, 3, 3, 4, 5, 1, 2, 3, 4, 1])
    mol = torch.tensor([0] * 11 + [const.MOL_NONPOLYMER])
    mask = torch.ones(12, dtype=torch.bool)
    h = plm(res_type, asym, resid, mol, mask)
    assert h.shape == (12, 4, 64) and h[-1].abs().sum() == 0
    assert torch.equal(h[2], h[3]) and torch.equal(h[3], h[4])  # atom tokens share their residue's states
    sel = asym == 1
    alone = plm(res_type[sel], asym[sel], resid[sel], mol[sel], mask[sel])
    assert torch.allclose(h[sel], alone, atol=1e-5)
    joined = FrozenPLM(cfg=_small_cfg(), join="joined")
    object.__setattr__(joined, "_backbone", plm._backbone)
    hj = joined(res_type, asym, resid, mol, mask)
    assert hj.shape == h.shape and not torch.allclose(hj[sel], alone, atol=1e-4)  # chains see each other
    assert "_backbone" not in dict(plm.named_modules()) and len(plm.state_dict()) == 0
    hb = plm(res_type[None], asym[None], resid[None], mol[None], mask[None])
    assert torch.allclose(hb[0], h)


def test_pair_shim_names_and_shapes():
    shim = LMPairShim(d_pair=16, d_model=64, num_layers=3)
    keys = set(shim.state_dict())
    assert {"layer_combine", "to_pair_channels.0.weight", "to_pair_channels.1.weight", "to_pair.0.downproject.weight",
            "to_pair.0.output_mlp.0.weight", "to_pair.0.output_mlp.2.bias", "to_pair.1.weight"} <= keys  # fmt: skip
    h = torch.randn(7, 4, 64)
    z = shim(h)
    assert z.shape == (7, 7, 16)
    with pytest.raises(ValueError):
        shim(torch.randn(7, 5, 64))
    z.sum().backward()
    assert shim.layer_combine.grad is not None
