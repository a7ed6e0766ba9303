"""tcgen05 GEMM kernel against an fp32 PyTorch statement of each epilogue."""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def df3():
    from deepfold3_dev_b200.ops import native

    native.require()
    return torch.ops.df3


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).bfloat16()


def _check(out, ref, tol=2e-2):
    assert out.shape == ref.shape
    err = (out.float() - ref).abs().max().item()
    mag = ref.abs().max().item() + 1e-6
    assert err <= tol * mag, f"max err {err} vs magnitude {mag}"


@pytest.mark.parametrize("rows,k,n", [(128, 64, 128), (1000, 128, 128), (4097, 384, 96), (333, 200, 16), (2048, 512, 384)])
def test_plain_bias_mask(df3, rows, k, n):
    x, w = _rand(rows, k, seed=1), _rand(n, k, seed=2, scale=k**-0.5)
    bias = torch.randn(n, device="cuda")
    mask = (torch.rand(rows, device="cuda") > 0.2).float()
    out = df3.gemm(x, w, bias, mask, None, 0, False)
    ref = (x.float() @ w.float().t() + bias) * mask[:, None]
    _check(out, ref)
    assert df3.gemm_status() == 0
    out2 = df3.gemm(x, w, None, None, None, 0, False)
    _check(out2, x.float() @ w.float().t())


def test_leading_axes_and_channel_major(df3):
    x, w = _rand(3, 50, 70, 128, seed=3), _rand(64, 128, seed=4, scale=0.1)
    out = df3.gemm(x, w, None, None, None, 0, False)
    _check(out, x.float() @ w.float().t())
    planes = df3.gemm(x, w, None, None, None, 0, True)
    _check(planes, (x.float() @ w.float().t()).reshape(-1, 64).t())


@pytest.mark.parametrize("rows,k,n", [(3000, 128, 256), (777, 128, 128), (500, 256, 64), (300, 64, 32)])
def test_gated_and_swiglu(df3, rows, k, n):
    x = _rand(rows, k, seed=5)
    wg, wp = _rand(n, k, seed=6, scale=k**-0.5), _rand(n, k, seed=7, scale=k**-0.5)
    w = torch.cat([wg, wp], 0)
    mask = (torch.rand(rows, device="cuda") > 0.2).float()
    g, p = x.float() @ wg.float().t(), x.float() @ wp.float().t()
    _check(df3.gemm(x, w, None, mask, None, 1, False), torch.sigmoid(g) * p * mask[:, None])
    _check(df3.gemm(x, w, None, None, None, 2, False), torch.nn.functional.silu(g) * p)
    _check(df3.gemm(x, w, None, None, None, 1, True), (torch.sigmoid(g) * p).t())
    assert df3.gemm_status() == 0


def test_sigmoid_mul(df3):
    x, w, o = _rand(900, 128, seed=8), _rand(128, 128, seed=9, scale=0.1), _rand(900, 128, seed=10)
    out = df3.gemm(x, w, None, None, o, 3, False)
    _check(out, torch.sigmoid(x.float() @ w.float().t()) * o.float())


def test_batched_nt(df3):
    a, b = _rand(6, 300, 384, seed=11, scale=0.1), _rand(6, 200, 384, seed=12, scale=0.1)
    _check(df3.bmm_nt(a, b), torch.einsum("bmk,bnk->bmn", a.float(), b.float()))
    assert df3.gemm_status() == 0
