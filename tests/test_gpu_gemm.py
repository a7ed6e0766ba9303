"""tcgen05 GEMM kernel against an fp32 PyTorch statement of each epilogue, element by element."""

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


def _check(out, ref, rtol=1e-2, atol_frac=1e-2):
    """|out - ref| <= atol + rtol |ref| for every element; atol is a fraction of the RMS of the expected values
    (bf16 outputs carry 2^-9 relative rounding; the accumulation itself is fp32)."""
    assert out.shape == ref.shape
    out, ref = out.float(), ref.float()
    atol = atol_frac * ref.pow(2).mean().sqrt().item() + 1e-30
    bad = (out - ref).abs() > atol + rtol * ref.abs()
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} off, worst {(out - ref).abs().max().item():.3e}, atol {atol:.3e}"


@pytest.mark.parametrize("rows,k,n", [(128, 64, 128), (1000, 128, 128), (4097, 384, 96), (333, 200, 16), (2048, 512, 384),
                                      (70000, 128, 128), (5000, 768, 768)])  # fmt: skip
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
    bias = torch.randn(64, device="cuda")
    mask = (torch.rand(3 * 50 * 70, device="cuda") > 0.3).float()
    planes = df3.gemm(x, w, bias, mask, None, 0, True)
    _check(planes, ((x.float() @ w.float().t() + bias).reshape(-1, 64) * mask[:, None]).t())
    assert df3.gemm_status() == 0


@pytest.mark.parametrize("rows,k,n", [(3000, 128, 256), (777, 128, 128), (500, 256, 64), (300, 64, 32), (20000, 128, 128)])
def test_gated_and_swiglu(df3, rows, k, n):
    x = _rand(rows, k, seed=5)
    wg, wp = _rand(n, k, seed=6, scale=k**-0.5), _rand(n, k, seed=7, scale=k**-0.5)
    w = torch.cat([wg, wp], 0)
    mask = (torch.rand(rows, device="cuda") > 0.2).float()
    g, p = x.float() @ wg.float().t(), x.float() @ wp.float().t()
    _check(df3.gemm(x, w, None, mask, None, 1, False), torch.sigmoid(g) * p * mask[:, None])
    _check(df3.gemm(x, w, None, None, None, 2, False), torch.nn.functional.silu(g) * p)
    _check(df3.gemm(x, w, None, None, None, 1, True), (torch.sigmoid(g) * p).t())
    _check(df3.gemm(x, w, None, mask, None, 1, True), (torch.sigmoid(g) * p * mask[:, None]).t())
    assert df3.gemm_status() == 0


def test_sigmoid_mul(df3):
    x, w, o = _rand(900, 128, seed=8), _rand(128, 128, seed=9, scale=0.1), _rand(900, 128, seed=10)
    out = df3.gemm(x, w, None, None, o, 3, False)
    _check(out, torch.sigmoid(x.float() @ w.float().t()) * o.float())
    x, w, o = _rand(3000, 768, seed=8), _rand(768, 768, seed=9, scale=0.03), _rand(3000, 768, seed=10)
    _check(df3.gemm(x, w, None, None, o, 3, False), torch.sigmoid(x.float() @ w.float().t()) * o.float())
    assert df3.gemm_status() == 0


def test_backward_epilogues(df3):
    rows, k, n = 1500, 128, 256
    x = _rand(rows, k, seed=20)
    wg, wp = _rand(n, k, seed=21, scale=k**-0.5), _rand(n, k, seed=22, scale=k**-0.5)
    w = torch.cat([wg, wp], 0)
    dy = _rand(rows, n, seed=23)
    mask = (torch.rand(rows, device="cuda") > 0.2).float()
    a, b = x.float() @ wg.float().t(), x.float() @ wp.float().t()
    s = torch.sigmoid(a)
    g = dy.float()
    out = df3.gemm(x, w, None, None, dy, 4, False)  # SwiGLU backward: [d pre-gate, d pre-proj]
    _check(out, torch.cat([g * b * s * (1 + a * (1 - s)), g * a * s], -1))
    out = df3.gemm(x, w, None, mask, dy, 5, False)  # gated backward
    gm = g * mask[:, None]
    _check(out, torch.cat([gm * b * s * (1 - s), gm * s], -1))
    assert df3.gemm_status() == 0


def test_batched_nt(df3):
    a, b = _rand(6, 300, 384, seed=11, scale=0.1), _rand(6, 200, 384, seed=12, scale=0.1)
    _check(df3.bmm_nt(a, b), torch.einsum("bmk,bnk->bmn", a.float(), b.float()))
    assert df3.gemm_status() == 0


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("B,M,N,K", [(1, 256, 128, 192), (5, 200, 136, 264), (3, 384, 384, 384), (1, 1000, 72, 1000)])
def test_matmul_operand_layouts(df3, trans_a, trans_b, B, M, N, K):
    """out = A B with either operand handed over transposed; no operand is copied."""
    a = _rand(B, K, M, seed=30, scale=K**-0.25) if trans_a else _rand(B, M, K, seed=30, scale=K**-0.25)
    b = _rand(B, N, K, seed=31, scale=K**-0.25) if trans_b else _rand(B, K, N, seed=31, scale=K**-0.25)
    A = a.float().transpose(1, 2) if trans_a else a.float()
    Bm = b.float().transpose(1, 2) if trans_b else b.float()
    ref = A @ Bm
    _check(df3.matmul(a, b, trans_a, trans_b, False, 1), ref)
    _check(df3.matmul(a, b, trans_a, trans_b, True, 1), ref, rtol=2e-3, atol_frac=2e-3)
    assert df3.gemm_status() == 0


def test_split_k_weight_gradient_is_reproducible(df3):
    """dW = dY^T X over many rows: split along K, partial sums added in a fixed order."""
    rows, n, k = 40000, 128, 128
    dy, x = _rand(rows, n, seed=40), _rand(rows, k, seed=41)
    ref = dy.float().t() @ x.float()
    out = df3.matmul(dy, x, True, False, True, 0)
    assert out.dtype == torch.float32
    _check(out, ref, rtol=2e-3, atol_frac=2e-3)
    assert torch.equal(out, df3.matmul(dy, x, True, False, True, 0))
    _check(df3.matmul(dy, x, True, False, True, 7), ref, rtol=2e-3, atol_frac=2e-3)
    dx_ref = dy.float() @ _rand(n, k, seed=42, scale=0.1).float()
    _check(df3.matmul(dy, _rand(n, k, seed=42, scale=0.1), False, False, False, 1), dx_ref)
    assert df3.gemm_status() == 0


def test_linear_bwd_on_own_kernels(df3):
    rows, n, k = 3000, 256, 128
    dy, x, w = _rand(7, rows // 7 + 1, n, seed=50), _rand(7, rows // 7 + 1, k, seed=51), _rand(n, k, seed=52, scale=0.1)
    dx, dw, db = df3.linear_bwd(dy, x, w, True, True, True)
    d2, x2 = dy.float().reshape(-1, n), x.float().reshape(-1, k)
    _check(dx, (d2 @ w.float()).view(x.shape))
    _check(dw, d2.t() @ x2, rtol=2e-3, atol_frac=2e-3)
    _check(db, d2.sum(0), rtol=2e-3, atol_frac=2e-3)
    assert df3.gemm_status() == 0
