"""Fused tcgen05 attention backward against the fp32 PyTorch statement, element by element.

Cases follow the reference's kernel robustness suite (tests/triton/test_evo_attn_robustness.py): logit magnitude
sweeps, heavy-tailed inputs, fully and nearly fully masked rows, token counts that are not multiples of the tile or of
8, every supported head width, strided (packed-projection) operands, and run-to-run bitwise reproducibility.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def df3():
    from deepfold3_dev_b200.ops import native

    native.require()
    return torch.ops.df3


def _reference_grads(q, k, v, bias, mask, scale, d_out):
    q32, k32, v32 = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    b32 = bias.float().detach().requires_grad_(True) if bias is not None else None
    s = torch.einsum("brhid,brhjd->brhij", q32, k32) * scale
    if b32 is not None:
        s = s + b32[:, None]
    if mask is not None:
        s = s + 1e9 * (mask.float()[:, :, None, None, :] - 1.0)
    p = torch.softmax(s, dim=-1)
    out = torch.einsum("brhij,brhjd->brhid", p, v32)
    out.backward(d_out.float())
    return q32.grad, k32.grad, v32.grad, (b32.grad if b32 is not None else None)


def _close(got, want, rtol, atol_frac, what):
    """Two checks against the fp32 statement. Every element: |got - want| <= atol + rtol |want|, atol a fraction of the
    RMS of the expected tensor (the kernel rounds P and dS to bf16 before the second-stage products, so one element
    carries the sum of up to N such roundings plus the bf16 rounding of the output). The tensor as a whole: relative
    RMS error below 1 %, which a systematic defect (a wrong scale, a missed tile) cannot meet."""
    got, want = got.float(), want.float()
    rms = want.pow(2).mean().sqrt().item() + 1e-30
    atol = 3 * atol_frac * rms
    err = (got - want).abs()
    bad = err > atol + rtol * want.abs()
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.numel()} elements off, worst {err.max().item():.3e} (atol {atol:.3e})"
    rel_rms = err.pow(2).mean().sqrt().item() / rms
    assert rel_rms < 1e-2, f"{what}: relative RMS error {rel_rms:.3e}"


def _run(df3, q, k, v, bias, mask, scale, d_out, chunked=False):
    out, lse, out32 = df3.attention_fwd_train(q, k, v, bias, mask, scale)
    dq, dk, dv, db = df3.attention_bwd(q, k, v, out if chunked else out32, d_out, bias, mask, lse, scale, bias is not None,
                                       -(40 << 20) if chunked else (40 << 20))
    assert df3.gemm_status() == 0
    return dq, dk, dv, db


def _inputs(B, R, H, N, D, seed, bias_dtype=torch.bfloat16, with_mask=True, qk_scale=1.0, bias_scale=2.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B, R, H, N, D, device="cuda", generator=g) for _ in range(3))
    q, k = (q * qk_scale).bfloat16(), (k * qk_scale).bfloat16()
    v = v.bfloat16()
    bias = (bias_scale * torch.randn(B, H, N, N, device="cuda", generator=g)).to(bias_dtype)
    mask = None
    if with_mask:
        mask = (torch.rand(B, R, N, device="cuda", generator=g) > 0.15).float()
        mask[..., 0] = 1.0
    d_out = torch.randn(B, R, H, N, D, device="cuda", generator=g).bfloat16()
    return q, k, v, bias, mask, d_out


SHAPES = [(1, 3, 4, 128, 32), (1, 2, 4, 384, 32), (2, 2, 2, 200, 64), (1, 1, 16, 384, 24), (1, 3, 16, 333, 48),
          (1, 2, 2, 520, 16), (1, 2, 4, 64, 32), (1, 2, 4, 77, 32), (1, 5, 4, 256, 16), (2, 3, 4, 136, 32)]  # fmt: skip


@pytest.mark.parametrize("B,R,H,N,D", SHAPES)
def test_fused_backward_matches_fp32_statement(df3, B, R, H, N, D):
    assert df3.attention_bwd_fused_supported(N, D)
    q, k, v, bias, mask, d_out = _inputs(B, R, H, N, D, seed=N + D)
    scale = D**-0.5
    got = _run(df3, q, k, v, bias, mask, scale, d_out)
    want = _reference_grads(q, k, v, bias, mask, scale, d_out)
    for g, w, name in zip(got, want, ("dq", "dk", "dv", "dbias")):
        _close(g, w, rtol=2e-2, atol_frac=2e-2, what=f"{name} {B, R, H, N, D}")


@pytest.mark.parametrize("bias_dtype", [torch.float32, torch.bfloat16])
def test_shared_bias_over_batch_and_no_mask(df3, bias_dtype):
    B, R, H, N, D = 2, 3, 4, 160, 32
    q, k, v, bias, _, d_out = _inputs(B, R, H, N, D, seed=11, bias_dtype=bias_dtype, with_mask=False)
    bias = bias[:1].contiguous()
    got = _run(df3, q, k, v, bias, None, D**-0.5, d_out)
    want = _reference_grads(q, k, v, bias, None, D**-0.5, d_out)
    for g, w, name in zip(got, want, ("dq", "dk", "dv", "dbias")):
        _close(g, w, rtol=2e-2, atol_frac=2e-2, what=name)


def test_no_bias(df3):
    B, R, H, N, D = 1, 4, 4, 192, 32
    q, k, v, _, mask, d_out = _inputs(B, R, H, N, D, seed=3)
    got = _run(df3, q, k, v, None, mask, D**-0.5, d_out)
    want = _reference_grads(q, k, v, None, mask, D**-0.5, d_out)
    for g, w, name in zip(got[:3], want[:3], ("dq", "dk", "dv")):
        _close(g, w, rtol=2e-2, atol_frac=2e-2, what=name)
    assert got[3].numel() == 0


@pytest.mark.parametrize("qk_scale", [1e-2, 0.3, 3.0, 10.0, 30.0])
def test_logit_magnitude_sweep(df3, qk_scale):
    """|q.k| / sqrt(D) from ~1e-4 to ~1e3: the recomputed probabilities keep matching the saved row statistics."""
    B, R, H, N, D = 1, 2, 4, 256, 32
    q, k, v, bias, mask, d_out = _inputs(B, R, H, N, D, seed=7, qk_scale=qk_scale)
    got = _run(df3, q, k, v, bias, mask, D**-0.5, d_out)
    want = _reference_grads(q, k, v, bias, mask, D**-0.5, d_out)
    for g, w, name in zip(got, want, ("dq", "dk", "dv", "dbias")):
        assert torch.isfinite(g.float()).all(), name
        _close(g, w, rtol=3e-2, atol_frac=3e-2, what=f"{name} at operand scale {qk_scale}")


def test_heavy_tailed_inputs(df3):
    B, R, H, N, D = 1, 2, 4, 256, 32
    g = torch.Generator(device="cuda").manual_seed(21)
    cauchy = lambda *s: torch.tan(3.14159 * (torch.rand(*s, device="cuda", generator=g) - 0.5)).clamp(-12, 12)  # noqa: E731
    q, k, v = (cauchy(B, R, H, N, D).bfloat16() for _ in range(3))
    bias = cauchy(B, H, N, N).bfloat16()
    d_out = cauchy(B, R, H, N, D).bfloat16()
    got = _run(df3, q, k, v, bias, None, D**-0.5, d_out)
    want = _reference_grads(q, k, v, bias, None, D**-0.5, d_out)
    for gg, w, name in zip(got, want, ("dq", "dk", "dv", "dbias")):
        assert torch.isfinite(gg.float()).all(), name
        _close(gg, w, rtol=3e-2, atol_frac=3e-2, what=name)


def test_fully_and_nearly_fully_masked_rows(df3):
    B, R, H, N, D = 1, 4, 4, 200, 32
    q, k, v, bias, mask, d_out = _inputs(B, R, H, N, D, seed=13)
    mask[:, 0] = 0.0          # every key of row 0 masked: uniform weights, finite gradients
    mask[:, 1] = 0.0
    mask[:, 1, 17] = 1.0      # one surviving key
    mask[:, 2, :192] = 0.0    # survivors only in the ragged last block
    got = _run(df3, q, k, v, bias, mask, D**-0.5, d_out)
    want = _reference_grads(q, k, v, bias, mask, D**-0.5, d_out)
    for g, w, name in zip(got, want, ("dq", "dk", "dv", "dbias")):
        assert torch.isfinite(g.float()).all(), name
        _close(g, w, rtol=2e-2, atol_frac=2e-2, what=name)


def test_run_twice_bitwise_identical(df3):
    B, R, H, N, D = 1, 6, 4, 384, 32
    q, k, v, bias, mask, d_out = _inputs(B, R, H, N, D, seed=5)
    a = _run(df3, q, k, v, bias, mask, D**-0.5, d_out)
    b = _run(df3, q, k, v, bias, mask, D**-0.5, d_out)
    for x, y, name in zip(a, b, ("dq", "dk", "dv", "dbias")):
        assert torch.equal(x, y), name


def test_fused_agrees_with_chunked_form(df3):
    B, R, H, N, D = 1, 5, 4, 264, 32
    q, k, v, bias, mask, d_out = _inputs(B, R, H, N, D, seed=9)
    a = _run(df3, q, k, v, bias, mask, D**-0.5, d_out)
    b = _run(df3, q, k, v, bias, mask, D**-0.5, d_out, chunked=True)
    for x, y, name in zip(a, b, ("dq", "dk", "dv", "dbias")):
        _close(x, y, rtol=3e-2, atol_frac=3e-2, what=name)


def test_gradients_written_into_packed_views(df3):
    """dq, dk, dv land in the three slots of a packed [B, N, N, 3, H, D] gradient (column attention views)."""
    B, N, H, D = 1, 136, 4, 32
    g = torch.Generator(device="cuda").manual_seed(2)
    qkv = torch.randn(B, N, N, 3, H, D, device="cuda", generator=g).bfloat16()
    heads = lambda t: t.permute(0, 2, 3, 1, 4)  # noqa: E731
    q, k, v = (heads(qkv[:, :, :, i]) for i in range(3))
    bias = torch.randn(B, H, N, N, device="cuda", generator=g).bfloat16()
    mask = (torch.rand(B, N, N, device="cuda", generator=g) > 0.1).float()
    mask[..., 0] = 1.0
    d_out = torch.randn(B, N, H, N, D, device="cuda", generator=g).bfloat16()
    out, lse, out32 = df3.attention_fwd_train(q, k, v, bias, mask, D**-0.5)
    assert torch.equal(out32.bfloat16(), out)
    dqkv = torch.full_like(qkv, float("nan"))
    dq, dk, dv = (heads(dqkv[:, :, :, i]) for i in range(3))
    db = df3.attention_bwd_into(q, k, v, out32, d_out, bias, mask, lse, D**-0.5, True, dq, dk, dv)
    assert df3.gemm_status() == 0
    assert torch.isfinite(dqkv.float()).all()
    want = _reference_grads(q, k, v, bias, mask, D**-0.5, d_out)
    for gg, w, name in zip((dq, dk, dv, db), want, ("dq", "dk", "dv", "dbias")):
        _close(gg, w, rtol=2e-2, atol_frac=2e-2, what=name)
