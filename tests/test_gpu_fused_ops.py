"""Forward values and gradients of the fused autograd ops against their eager fp32 statements."""

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    from deepfold3_dev_b200.ops import native

    return native.require()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def _leaf(*shape, seed, scale=1.0, dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype).requires_grad_(True)


def _compare(fused_fn, eager_fn, inputs, tol=3e-2):
    """Runs both on clones of ``inputs`` (fused gets bf16 activations where eager gets fp32) and compares."""
    outs = []
    for fn in (fused_fn, eager_fn):
        leaves = [t.detach().clone().requires_grad_(t.requires_grad) for t in inputs]
        y = fn(*leaves)
        g = torch.Generator(device="cuda").manual_seed(99)
        w = torch.randn(y.shape, device="cuda", generator=g)
        (y.float() * w).sum().backward()
        outs.append((y.detach(), [t.grad for t in leaves]))
    (yf, gf), (ye, ge) = outs
    assert _rel(yf, ye) < tol, f"forward {_rel(yf, ye)}"
    for i, (a, b) in enumerate(zip(gf, ge)):
        if b is None:
            continue
        assert a is not None, f"missing grad {i}"
        assert _rel(a, b) < tol, f"grad of input {i}: {_rel(a, b)}"


@pytest.mark.parametrize("planes,deint", [(False, False), (True, False), (True, True)])
def test_gated_dual(nat, planes, deint):
    x = _leaf(500, 64, seed=1)
    wg, wp = _leaf(48, 64, seed=2, scale=0.2), _leaf(48, 64, seed=3, scale=0.2)
    mask = (torch.rand(500, device="cuda") > 0.3).float()

    def eager(x, wg, wp):
        xb = x.bfloat16().float()
        y = torch.sigmoid(xb @ wg.bfloat16().float().t()) * (xb @ wp.bfloat16().float().t()) * mask[:, None]
        if deint:
            y = torch.cat([y[:, 0::2], y[:, 1::2]], -1)
        return y.t() if planes else y

    _compare(lambda x, wg, wp: nat.gated_dual_linear(x, wg, wp, mask, planes, deint), eager, [x, wg, wp])


def test_linear_planes_sigmoid_gate_stacked(nat):
    x = _leaf(3, 40, 64, seed=4)
    w = _leaf(8, 64, seed=5, scale=0.2)
    _compare(lambda x, w: nat.linear_planes(x, w), lambda x, w: F.linear(x, w).reshape(-1, 8).t(), [x, w])
    wg = _leaf(32, 64, seed=6, scale=0.2)
    other = _leaf(3, 40, 32, seed=7)
    _compare(lambda x, w, o: nat.sigmoid_gate_mul(x, w, o), lambda x, w, o: torch.sigmoid(F.linear(x, w)) * o, [x, wg, other])
    w2, w3 = _leaf(16, 64, seed=8, scale=0.2), _leaf(24, 64, seed=9, scale=0.2)
    _compare(lambda x, a, b, c: nat.stacked_linear(x, a, b, c),
             lambda x, a, b, c: torch.cat([F.linear(x, a), F.linear(x, b), F.linear(x, c)], -1), [x, w, w2, w3])  # fmt: skip


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_transition(nat, dtype):
    x = _leaf(700, 64, seed=10, dtype=dtype)
    lw, lb = _leaf(64, seed=11), _leaf(64, seed=12, scale=0.1)
    w1, w2 = _leaf(256, 64, seed=13, scale=0.15), _leaf(64, 128, seed=14, scale=0.1)

    def eager(x, lw, lb, w1, w2):
        h = F.layer_norm(x.float(), (64,), lw, lb)
        a, b = F.linear(h, w1).chunk(2, -1)
        return F.linear(F.silu(a) * b, w2)

    _compare(lambda *a: nat.transition(*a, 1e-5), eager, [x, lw, lb, w1, w2], tol=4e-2)


@pytest.mark.parametrize("B,R,H,N,D,column", [(1, 5, 4, 136, 16, False), (1, 136, 2, 136, 32, True), (2, 3, 4, 200, 24, False)])
def test_attention_gradients(nat, B, R, H, N, D, column):
    g = torch.Generator(device="cuda").manual_seed(N)
    if column:  # strided views of a fused projection, column flavour
        proj = _leaf(B, N, R, 3 * H * D, seed=20, dtype=torch.bfloat16)
    else:
        proj = _leaf(B, R, N, 3 * H * D, seed=20, dtype=torch.bfloat16)
    bias = _leaf(B, H, N, N, seed=21, dtype=torch.bfloat16)
    mask = (torch.rand(B, R, N, device="cuda", generator=g) > 0.2).float()
    mask[:, 0] = 0  # one row with every key masked: uniform weights, finite gradients

    def split(proj):
        t = proj.view(*proj.shape[:3], 3, H, D)
        qkv = [t[:, :, :, i] for i in range(3)]
        perm = (0, 2, 3, 1, 4) if column else (0, 1, 3, 2, 4)
        return [u.permute(*perm) for u in qkv]

    def fused(proj, bias):
        q, k, v = split(proj)
        return nat.pair_bias_attention(q, k, v, bias, mask, D**-0.5)

    def eager(proj, bias):
        q, k, v = (u.float() for u in split(proj))
        s = q @ k.transpose(-1, -2) * D**-0.5 + bias.float()[:, None] + 1e9 * (mask[:, :, None, None, :] - 1)
        return torch.softmax(s, -1) @ v

    _compare(fused, eager, [proj, bias], tol=4e-2)
    assert torch.ops.df3.gemm_status() == 0


@pytest.mark.parametrize("outgoing", [True, False])
def test_triangle_projection_contract(outgoing):
    from deepfold3_dev_b200 import ops

    N, C = 72, 32
    z0 = _leaf(1, N, N, C, seed=30, dtype=torch.bfloat16)
    wg, wp = _leaf(2 * C, C, seed=31, scale=0.3), _leaf(2 * C, C, seed=32, scale=0.3)
    mask = (torch.rand(1, N, N, device="cuda") > 0.1).float()

    def eager(z0, wg, wp):
        x = z0.float()
        ab = torch.sigmoid(x @ wg.bfloat16().float().t()) * (x @ wp.bfloat16().float().t()) * mask[..., None]
        a, b = ab[..., 0::2], ab[..., 1::2]
        return torch.einsum("bikc,bjkc->bijc", a, b) if outgoing else torch.einsum("bkjc,bkic->bijc", a, b)

    _compare(lambda z0, wg, wp: ops.triangle_projection_contract(z0, wg, wp, mask, outgoing), eager, [z0, wg, wp], tol=4e-2)


@pytest.mark.parametrize("C,M", [(128, 5000), (32, 777), (64, 64)])
def test_plane_layer_norm(nat, C, M):
    x = _leaf(C, M, seed=40, dtype=torch.bfloat16)
    w, b = _leaf(C, seed=41), _leaf(C, seed=42, scale=0.1)
    _compare(lambda x, w, b: nat.plane_layer_norm(x, w, b, 1e-5),
             lambda x, w, b: F.layer_norm(x.float().t(), (C,), w, b), [x, w, b], tol=3e-2)


@pytest.mark.parametrize("ta,tb", [(False, False), (False, True), (True, False), (True, True)])
def test_differentiable_matmul_layouts(nat, ta, tb):
    B, M, N, K = 3, 136, 72, 200
    a = _leaf(B, K, M, seed=11, scale=0.2) if ta else _leaf(B, M, K, seed=11, scale=0.2)
    b = _leaf(B, N, K, seed=12, scale=0.2) if tb else _leaf(B, K, N, seed=12, scale=0.2)

    def eager(a, b):
        A = a.bfloat16().float()
        Bm = b.bfloat16().float()
        return (A.transpose(1, 2) if ta else A) @ (Bm.transpose(1, 2) if tb else Bm)

    _compare(lambda a, b: nat.matmul(a.bfloat16(), b.bfloat16(), ta, tb), eager, [a, b])


def test_msa_weighted_average_and_outer_product_mean(nat):
    from deepfold3_dev_b200 import ops
    from deepfold3_dev_b200.ops import reference as ref

    B, S, N, H, D = 1, 40, 72, 8, 8
    w = torch.softmax(_leaf(B, H, N, N, seed=21).detach(), -1).requires_grad_(True)
    v = _leaf(B, S, N, H, D, seed=22)
    _compare(lambda w, v: ops.msa_weighted_average(w.bfloat16(), v.bfloat16()),
             lambda w, v: ref.msa_weighted_average(w.bfloat16().float(), v.bfloat16().float()), [w, v])
    E, C = 32, 128
    a, b = _leaf(B, S, N, E, seed=23, scale=0.5), _leaf(B, S, N, E, seed=24, scale=0.5)
    out_w, out_b = _leaf(E, E, C, seed=25, scale=0.05), _leaf(C, seed=26)
    mask = (torch.rand(B, S, N, device="cuda") > 0.2).float()
    ops.census(reset=True)
    _compare(lambda a, b, ow, ob: ops.outer_product_mean((a * mask[..., None]).bfloat16(), (b * mask[..., None]).bfloat16(), ow, ob, mask),
             lambda a, b, ow, ob: ref.outer_product_mean((a * mask[..., None]).bfloat16().float(), (b * mask[..., None]).bfloat16().float(),
                                                         ow.bfloat16().float(), ob, mask), [a, b, out_w, out_b], tol=4e-2)
    c = ops.census()
    assert c.get("outer_product_mean:sm100", 0) == 1 and c.get("msa_weighted_average:sm100", 0) == 0  # census was reset in between
    assert torch.ops.df3.gemm_status() == 0
