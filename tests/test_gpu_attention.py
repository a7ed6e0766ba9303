"""tcgen05 pair-bias attention forward against the fp32 PyTorch statement."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def df3():
    from deepfold3_dev_b200.ops import native

    native.require()
    return torch.ops.df3


def _reference(q, k, v, bias, mask, scale):
    s = torch.einsum("brhid,brhjd->brhij", q.float(), k.float()) * scale
    if bias is not None:
        s = s + bias.float()[:, None]
    if mask is not None:
        s = s + 1e9 * (mask.float()[:, :, None, None, :] - 1.0)
    p = torch.softmax(s, dim=-1)
    return torch.einsum("brhij,brhjd->brhid", p, v.float()), torch.logsumexp(s, dim=-1)


def _inputs(B, R, H, N, D, seed, bias_dtype=torch.bfloat16, with_mask=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B, R, H, N, D, device="cuda", generator=g).bfloat16() for _ in range(3))
    bias = (2 * torch.randn(B, H, N, N, device="cuda", generator=g)).to(bias_dtype)
    mask = None
    if with_mask:
        mask = (torch.rand(B, R, N, device="cuda", generator=g) > 0.15).float()
        mask[..., 0] = 1.0
    return q, k, v, bias, mask


@pytest.mark.parametrize("B,R,H,N,D", [(1, 3, 4, 128, 32), (1, 2, 4, 384, 32), (2, 2, 2, 200, 64), (1, 1, 16, 384, 24),
                                       (1, 3, 16, 333, 48), (1, 2, 2, 520, 16)])  # fmt: skip
def test_matches_reference(df3, B, R, H, N, D):
    q, k, v, bias, mask = _inputs(B, R, H, N, D, seed=N + D)
    scale = D**-0.5
    out, lse = df3.attention_fwd(q, k, v, bias, mask, scale, True)
    assert df3.gemm_status() == 0
    ref, ref_lse = _reference(q, k, v, bias, mask, scale)
    assert (out.float() - ref).abs().max().item() < 3e-2
    assert ((lse[0] + lse[1]) / 1.4426950408889634 - ref_lse).abs().max().item() < 2e-2


def test_strided_views_no_bias_fp32_bias(df3):
    B, N1, N2, H, D = 1, 160, 160, 4, 32
    g = torch.Generator(device="cuda").manual_seed(5)
    proj = torch.randn(B, N1, N2, 3 * H * D, device="cuda", generator=g).bfloat16()
    q, k, v = (t.view(B, N1, N2, H, D) for t in proj.split(H * D, dim=-1))
    # column attention: the independent axis is N2, the sequence axis N1
    qc, kc, vc = (t.permute(0, 2, 3, 1, 4) for t in (q, k, v))
    out, _ = df3.attention_fwd(qc, kc, vc, None, None, D**-0.5, False)
    ref, _ = _reference(qc, kc, vc, None, None, D**-0.5)
    assert (out.float() - ref).abs().max().item() < 3e-2
    bias = torch.randn(B, H, N1, N1, device="cuda", generator=g)
    out, _ = df3.attention_fwd(qc, kc, vc, bias, None, D**-0.5, False)
    ref, _ = _reference(qc, kc, vc, bias, None, D**-0.5)
    assert (out.float() - ref).abs().max().item() < 3e-2
    assert df3.gemm_status() == 0
