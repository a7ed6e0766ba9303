"""AF3 parameter name map: round trip through the Haiku layout, and agreement with the reference's converter."""

import numpy as np
import pytest
import torch

from deepfold3_dev_b200.config import schema as MC
from deepfold3_dev_b200.convert import af3
from deepfold3_dev_b200.convert.af3_name_map import BY_SCOPE
from deepfold3_dev_b200.models.model import DeepFold3
from tests.helpers import small_full_width


@pytest.fixture(scope="module")
def state():
    torch.manual_seed(0)
    model = DeepFold3(small_full_width(MC))
    sd = {k: torch.randn_like(v) for k, v in model.state_dict().items() if v.is_floating_point()}
    return model, sd


def test_round_trip_covers_the_model(state):
    model, sd = state
    params = af3.torch_to_haiku(sd)
    back = af3.haiku_to_torch(params)
    # everything AF3 publishes: all parameters except buffers that AF3 keeps as source constants (Fourier features)
    # and modules AF3 does not have
    missing = sorted(k for k in sd if k not in back)
    allowed = ("fourier_", "masked_msa_head.", "branch_scaler", "null_pair", "pair_bias_gate", "half_logits_ln", "router")
    assert all(any(a in k for a in allowed) for k in missing), missing[:20]
    for k, v in back.items():
        torch.testing.assert_close(v, sd[k].float(), atol=0, rtol=0)
    result = model.load_state_dict(back, strict=False)
    assert not result.unexpected_keys


def test_agrees_with_reference_converter(state, reference_package):
    from deepfold3.convert.af3 import haiku_to_torch as reference_convert

    _, sd = state
    params = af3.torch_to_haiku(sd)
    # the published layout keeps the output axes of multi-head projections apart: [in, heads, dim]
    w = params["diffuser/evoformer/__layer_stack_no_per_layer_1/trunk_pairformer/pair_attention1/v_projection"]["weights"]
    params["diffuser/evoformer/__layer_stack_no_per_layer_1/trunk_pairformer/pair_attention1/v_projection"]["weights"] = w.reshape(
        w.shape[0], w.shape[1], 4, -1)
    ref = reference_convert(params)
    mine = af3.haiku_to_torch(params)
    assert set(ref) == set(mine), sorted(set(ref) ^ set(mine))[:20]
    for k in ref:
        torch.testing.assert_close(mine[k], ref[k], atol=0, rtol=0)


def test_scope_names_are_unique_and_reader_round_trips(tmp_path, state):
    import struct

    assert len(BY_SCOPE) > 300
    _, sd = state
    params = af3.torch_to_haiku(sd)
    path = tmp_path / "af3.bin"
    with open(path, "wb") as f:
        for scope, arrays in list(params.items())[:40]:
            for name, arr in arrays.items():
                arr = np.ascontiguousarray(arr, dtype=np.float32)
                s, n, d = scope.encode(), name.encode(), b"float32"
                f.write(struct.pack("<5i", len(s), len(n), len(d), arr.ndim, arr.nbytes))
                f.write(struct.pack(f"<{len(s)}s{len(n)}s{len(d)}s{arr.ndim}i", s, n, d, *arr.shape))
                f.write(arr.tobytes())
    back = af3.read_af3_params(str(path))
    first = next(iter(back))
    np.testing.assert_array_equal(next(iter(back[first].values())), next(iter(params[first].values())))
    assert set(af3.convert_file(str(path))) <= set(sd)
