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


@pytest.mark.gpu
@pytest.mark.parametrize("transpose", [False, True])
def test_grid_attention_packed_gradients(transpose, monkeypatch):
    """The packed-projection path gives the gradients of the three-slice path and of the fp32 statement."""
    import torch

    from deepfold3_dev_b200 import ops
    from deepfold3_dev_b200.ops import reference as ref

    torch.manual_seed(0)
    B, N, H, D = 1, 64, 4, 32
    qkv0 = torch.randn(B, N, N, 3, H, D, device="cuda")
    bias0 = torch.randn(B, H, N, N, device="cuda")
    mask = (torch.rand(B, N, N, device="cuda") > 0.1).float()
    w = torch.randn(B, N, H, N, D, device="cuda")

    def run(packed: bool, fp32: bool = False):
        monkeypatch.setenv("DF3_DISABLE_OPS", "" if packed else "grid_attention_packed")
        qkv = (qkv0.clone() if fp32 else qkv0.bfloat16()).requires_grad_(True)
        bias = (bias0.clone() if fp32 else bias0.bfloat16()).requires_grad_(True)
        if fp32:
            heads = (lambda t: t.permute(0, 2, 3, 1, 4)) if transpose else (lambda t: t.permute(0, 1, 3, 2, 4))
            out = ref.pair_bias_attention(heads(qkv[:, :, :, 0]), heads(qkv[:, :, :, 1]), heads(qkv[:, :, :, 2]), bias, mask, D**-0.5)
        else:
            out = ops.grid_attention(qkv, bias, mask, D**-0.5, transpose)
        (out.float() * w).sum().backward()
        return out.float().detach(), qkv.grad.float(), bias.grad.float()

    ops.census(reset=True)
    o1, g1, b1 = run(True)
    o2, g2, b2 = run(False)
    o3, g3, b3 = run(True, fp32=True)
    assert ops.census().get("pair_bias_attention:sm100", 0) == 2
    assert torch.equal(o1, o2) and torch.allclose(g1, g2, atol=1e-6) and torch.allclose(b1, b2, atol=1e-6)
    for got, want in ((o1, o3), (g1, g3), (b1, b3)):
        assert (got - want).abs().max() <= 0.03 * want.abs().max() + 1e-3


@pytest.mark.parametrize("bias_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("S,W,Q,K,D", [(3, 5, 32, 128, 32), (2, 7, 32, 128, 16), (1, 3, 24, 72, 32), (2, 2, 160, 264, 32)])
def test_window_attention_matches_reference(df3, bias_dtype, S, W, Q, K, D):
    """Atom-window attention (few queries against more keys, bias per window shared by the samples, key mask folded
    into the bias) through ``ops.window_attention`` against the fp32 statement; rows of a fully masked window stay finite."""
    from deepfold3_dev_b200 import ops
    from deepfold3_dev_b200.ops import reference as ref

    H, B = 4, 1
    g = torch.Generator(device="cuda").manual_seed(S * 100 + W)
    # the model's layout: projections [B, S, W, tokens, H, D] with heads moved in front of tokens as a view
    q = torch.randn(B, S, W, Q, H, D, device="cuda", generator=g).bfloat16().transpose(-2, -3)
    k = torch.randn(B, S, W, K, H, D, device="cuda", generator=g).bfloat16().transpose(-2, -3)
    v = torch.randn(B, S, W, K, H, D, device="cuda", generator=g).bfloat16().transpose(-2, -3)
    keep = torch.rand(B, 1, W, 1, 1, K, device="cuda", generator=g) > 0.2
    keep[..., 0] = True
    keep[:, :, W - 1] = False  # one window without any live key
    bias = (2 * torch.randn(B, 1, W, H, Q, K, device="cuda", generator=g) + 1e9 * (keep.float() - 1.0)).to(bias_dtype)
    ops.census(reset=True)
    with torch.no_grad():
        out = ops.window_attention(q, k, v, bias, D**-0.5)
    assert ops.census().get("window_attention:sm100", 0) == 1
    want = ref.window_attention(q.float(), k.float(), v.float(), bias.float(), D**-0.5)
    assert out.shape == want.shape and torch.isfinite(out.float()).all()
    live = slice(0, W - 1)
    err = (out.float() - want)[:, :, live].abs().max().item()
    assert err < 0.03, err
    # a window with every key masked gives the plain mean of v over the keys (all logits equal), like the statement
    assert (out.float() - want)[:, :, W - 1].abs().max().item() < 0.05
    # the output's memory order follows q, so the model's reshape to [B, S, W, Q, H * D] is a view
    assert out.transpose(-2, -3).reshape(B, S, W, Q, H * D).data_ptr() == out.data_ptr()
    # with gradients wanted the forward-only kernel is not used
    ops.census(reset=True)
    ops.window_attention(q.clone().requires_grad_(True), k, v, bias, D**-0.5)
    assert ops.census().get("window_attention:sm100", 0) == 0


@pytest.mark.parametrize("S,W,Q,K,D", [(3, 5, 32, 128, 32), (2, 3, 24, 72, 16)])
def test_window_attention_gradients(df3, S, W, Q, K, D, monkeypatch):
    """Training path of the atom-window attention (queries padded to the key count, training forward + fused backward):
    output and the gradients of q, k, v and of the bias (summed over the samples) against the fp32 statement."""
    from deepfold3_dev_b200 import ops
    from deepfold3_dev_b200.ops import reference as ref

    monkeypatch.setenv("DF3_WINDOW_ATTENTION_TRAIN", "1")  # the kernels are opt-in for training (the default is the statement)
    H, B = 4, 1
    g = torch.Generator(device="cuda").manual_seed(7 * S + W)
    mk = lambda n: torch.randn(B, S, W, n, H, D, device="cuda", generator=g).bfloat16()  # noqa: E731
    q0, k0, v0 = mk(Q), mk(K), mk(K)
    keep = torch.rand(B, 1, W, 1, 1, K, device="cuda", generator=g) > 0.2
    keep[..., 0] = True
    b0 = (torch.randn(B, 1, W, H, Q, K, device="cuda", generator=g) + 1e9 * (keep.float() - 1.0)).bfloat16()
    w = torch.randn(B, S, W, H, Q, D, device="cuda", generator=g)

    def run(fn, cast):
        leaves = [t.detach().clone().to(cast).requires_grad_(True) for t in (q0, k0, v0, b0)]
        q, k, v, b = leaves
        out = fn(q.transpose(-2, -3), k.transpose(-2, -3), v.transpose(-2, -3), b, D**-0.5)
        (out.float() * w).sum().backward()
        return out.detach().float(), [t.grad.float() for t in leaves]

    ops.census(reset=True)
    out, grads = run(ops.window_attention, torch.bfloat16)
    assert ops.census().get("window_attention_train:sm100", 0) == 1
    want, want_grads = run(ref.window_attention, torch.float32)
    assert (out - want).abs().max().item() < 0.03
    for got, ref_g, name in zip(grads, want_grads, "qkvb"):
        scale = ref_g.abs().max().item()
        assert torch.isfinite(got).all() and (got - ref_g).abs().max().item() < 0.03 * scale + 2e-2, (name, (got - ref_g).abs().max().item(), scale)
