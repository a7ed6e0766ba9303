"""Safety nets around the kernels: guard bands around outputs that a kernel writes in place, bitwise repeatability of
every reduction whose order the kernels fix, and a dispatch-level check that a bf16 Pairformer block reaches no
library matrix product in forward or backward."""

import pytest
import torch

pytestmark = pytest.mark.gpu

SENTINEL = 12345.0


def guarded(shape, dtype=torch.bfloat16, pad=4096):
    """A contiguous tensor of ``shape`` cut out of a larger buffer filled with a sentinel, and a function that checks
    that nothing outside the tensor was written."""
    n = 1
    for d in shape:
        n *= d
    buf = torch.full((n + 2 * pad,), SENTINEL, dtype=dtype, device="cuda")
    view = buf[pad : pad + n].view(*shape)

    def check():
        assert bool((buf[:pad] == SENTINEL).all()) and bool((buf[pad + n :] == SENTINEL).all()), "write outside the output"

    return view, check


@pytest.fixture(scope="module")
def nat():
    from deepfold3_dev_b200.ops import native

    return native.require()


@pytest.mark.parametrize("M,N,K", [(200, 136, 72), (128, 128, 64), (1000, 264, 40)])
def test_matmul_stays_inside_a_preallocated_output(nat, M, N, K):
    a = torch.randn(3, M, K, device="cuda").bfloat16()
    b = torch.randn(3, K, N, device="cuda").bfloat16()
    out, check = guarded((3, M, N))
    torch.ops.df3.matmul(a, b, False, False, False, 1, out)
    torch.cuda.synchronize()
    check()
    torch.testing.assert_close(out.float(), torch.bmm(a.float(), b.float()), atol=0.15, rtol=2e-2)
    out32, check32 = guarded((3, M, N), torch.float32)
    torch.ops.df3.matmul(a, b, False, False, True, 1, out32)
    torch.cuda.synchronize()
    check32()


@pytest.mark.parametrize("N,D", [(72, 32), (200, 24), (384, 32)])
def test_attention_backward_stays_inside_its_outputs_and_repeats_bitwise(nat, N, D):
    B, R, H = 1, 5, 4
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v = (torch.randn(B, R, H, N, D, device="cuda", generator=g).bfloat16() for _ in range(3))
    bias = torch.randn(B, H, N, N, device="cuda", generator=g).bfloat16()
    mask = (torch.rand(B, R, N, device="cuda", generator=g) > 0.1).float()
    mask[:, :, 0] = 1
    out, lse, out32 = torch.ops.df3.attention_fwd_train(q, k, v, bias, mask, D**-0.5)
    d_out = torch.randn(out.shape, device="cuda", generator=g).bfloat16()
    if not torch.ops.df3.attention_bwd_fused_supported(N, D):
        pytest.skip("beyond the fused kernel's tensor-memory budget")
    runs = []
    for _ in range(2):
        bufs = [guarded((B, R, H, N, D)) for _ in range(3)]
        dbias = torch.ops.df3.attention_bwd_into(q, k, v, out32, d_out, bias, mask, lse, D**-0.5, True, *(b[0] for b in bufs))
        torch.cuda.synchronize()
        for _, check in bufs:
            check()
        runs.append([b[0].clone() for b in bufs] + [dbias.clone()])
    for a, b in zip(*runs):
        assert torch.equal(a, b)  # dq, dk, dv and the bias gradient: no atomics, fixed order
    assert torch.ops.df3.gemm_status() == 0


def test_weight_gradients_and_norm_backward_repeat_bitwise(nat):
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(5000, 128, device="cuda", generator=g).bfloat16()
    dy = torch.randn(5000, 256, device="cuda", generator=g).bfloat16()
    a = torch.ops.df3.matmul(dy, x, True, False, True, 0)   # split along the rows, partial sums added in a fixed order
    b = torch.ops.df3.matmul(dy, x, True, False, True, 0)
    assert torch.equal(a, b)
    w = torch.randn(128, device="cuda", generator=g)
    y, mean, rstd = torch.ops.df3.layer_norm_fwd(x, w, w, 1e-5)
    r1 = torch.ops.df3.layer_norm_bwd(y, x, w, mean, rstd, True)
    r2 = torch.ops.df3.layer_norm_bwd(y, x, w, mean, rstd, True)
    assert all(torch.equal(p, q) for p, q in zip(r1, r2))
    planes = torch.randn(128, 4104, device="cuda", generator=g).bfloat16()
    p1 = torch.ops.df3.plane_layer_norm_fwd(planes, w, w, 1e-5)
    p2 = torch.ops.df3.plane_layer_norm_fwd(planes, w, w, 1e-5)
    assert all(torch.equal(p, q) for p, q in zip(p1, p2))


def test_pairformer_block_reaches_no_library_matrix_product(nat):
    """bf16 forward and backward of a full-width Pairformer block: every matrix product runs on this package's GEMM
    and attention kernels (the dispatcher sees no aten mm / bmm / addmm / baddbmm / linear / matmul / sdpa call)."""
    from torch.utils._python_dispatch import TorchDispatchMode

    from deepfold3_dev_b200.models.evoformer import PairFormerBlock
    from tests.helpers import wake_zero_init

    torch.manual_seed(0)
    block = PairFormerBlock(128, 384).cuda().train()
    wake_zero_init(block)
    N = 128
    pair = torch.randn(1, N, N, 128, device="cuda", requires_grad=True)
    single = torch.randn(1, N, 384, device="cuda", requires_grad=True)
    seq_mask = torch.ones(1, N, device="cuda")
    pair_mask = torch.ones(1, N, N, device="cuda")
    seen, where = set(), {}
    keys = ("aten.mm", "aten.bmm", "aten.addmm", "aten.baddbmm", "aten.linear", "aten.matmul", "scaled_dot_product", "aten._addmm")

    class Watch(TorchDispatchMode):
        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            name = str(func)
            seen.add(name)
            if any(k in name for k in keys) and name not in where:
                import traceback

                where[name] = [f"{f.filename.split('/')[-1]}:{f.lineno}" for f in traceback.extract_stack() if "deepfold3_dev_b200" in f.filename][-4:]
            return func(*args, **(kwargs or {}))

    with Watch(), torch.autocast("cuda", dtype=torch.bfloat16):
        p, s = block(pair, single, pair_mask, seq_mask)
        (p.float().square().mean() + s.float().square().mean()).backward()
    library = {name for name in seen if any(key in name for key in keys)}
    assert not library, f"library matrix products reached: {where}"
    assert any("df3" in name for name in seen)
    assert pair.grad is not None and bool(torch.isfinite(pair.grad).all())


def test_bounds_checked_build_runs_the_same_ops_clean(tmp_path):
    """The debug build (index tests around the kernels' computed global accesses) computes the same results and its
    status words stay 0 on shapes with ragged edges. Needs ``python -m deepfold3_dev_b200.ops.build --checked``."""
    import os
    import subprocess
    import sys

    from deepfold3_dev_b200.ops import build as ops_build

    if not os.path.exists(ops_build.CHECKED_SO_PATH):
        pytest.skip("the checked extension has not been built")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = """
import torch
from deepfold3_dev_b200.ops import native
nat = native.require()
assert torch.ops.df3.bounds_checked()
x = torch.randn(5000, 128, device="cuda").bfloat16()
w = torch.randn(136, 128, device="cuda").bfloat16() * 0.1
y = torch.ops.df3.gemm(x, w, None, None, None, 0, False)
torch.testing.assert_close(y.float(), x.float() @ w.float().t(), atol=0.1, rtol=2e-2)
g = torch.ones(128, device="cuda")
n = torch.ops.df3.layer_norm_fwd(x, g, g, 1e-5)[0]
torch.testing.assert_close(n.float(), torch.nn.functional.layer_norm(x.float(), (128,), g, g), atol=3e-2, rtol=2e-2)
planes = torch.randn(128, 5000, device="cuda").bfloat16()
p = torch.ops.df3.plane_layer_norm_fwd(planes, g, g, 1e-5)[0]
torch.testing.assert_close(p.float(), torch.nn.functional.layer_norm(planes.float().t(), (128,), g, g), atol=3e-2, rtol=2e-2)
torch.cuda.synchronize()
assert torch.ops.df3.gemm_status() == 0 and torch.ops.df3.elementwise_status() == 0
print("CHECKED_OK")
"""
    env = dict(os.environ, DF3_BOUNDS_CHECK="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "CHECKED_OK" in out.stdout, out.stdout[-2000:] + out.stderr[-2000:]


# ---- forward attention and fused epilogues on hard inputs (cases after the reference's robustness suites for its
# ---- fused attention and fused modules: magnitude sweeps, heavy tails, masked rows, head widths, ragged lengths)
def _attention_reference(q, k, v, bias, mask, scale):
    s = torch.einsum("brhid,brhjd->brhij", q.float(), k.float()) * scale
    if bias is not None:
        s = s + bias.float()[:, None]
    if mask is not None:
        s = s + 1e9 * (mask.float()[:, :, None, None, :] - 1.0)
    return torch.einsum("brhij,brhjd->brhid", torch.softmax(s, dim=-1), v.float())


def _close(got, want, atol, rtol):
    torch.testing.assert_close(got.float(), want.float(), atol=atol, rtol=rtol)


@pytest.mark.parametrize("D", [16, 24, 32, 48, 64])
@pytest.mark.parametrize("N", [197, 264])
def test_attention_forward_head_widths_and_ragged_lengths(nat, D, N):
    g = torch.Generator(device="cuda").manual_seed(D + N)
    q, k, v = (torch.randn(1, 3, 4, N, D, device="cuda", generator=g).bfloat16() for _ in range(3))
    bias = torch.randn(1, 4, N, N, device="cuda", generator=g).bfloat16()
    mask = (torch.rand(1, 3, N, device="cuda", generator=g) > 0.2).float()
    mask[..., 0] = 1
    out, _ = torch.ops.df3.attention_fwd(q, k, v, bias, mask, D**-0.5, False)
    _close(out, _attention_reference(q, k, v, bias, mask, D**-0.5), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("magnitude", [1e-2, 1.0, 30.0, 300.0, 1000.0])
def test_attention_forward_logit_magnitude_sweep(nat, magnitude):
    """From nearly uniform rows to rows where one key takes everything (|logit| up to 1000: the running maximum and the
    rescaling have to carry it; a plain exp would overflow at 89)."""
    g = torch.Generator(device="cuda").manual_seed(3)
    N, D = 256, 32
    q, k, v = (torch.randn(1, 2, 4, N, D, device="cuda", generator=g).bfloat16() for _ in range(3))
    bias = (magnitude * torch.randn(1, 4, N, N, device="cuda", generator=g)).bfloat16()
    out, _ = torch.ops.df3.attention_fwd(q, k, v, bias, None, D**-0.5, False)
    assert bool(torch.isfinite(out).all())
    _close(out, _attention_reference(q, k, v, bias, None, D**-0.5), atol=3e-2, rtol=3e-2)


def test_attention_forward_heavy_tails_and_masked_rows(nat):
    g = torch.Generator(device="cuda").manual_seed(4)
    N, D = 200, 32
    q, k, v = (torch.randn(1, 4, 4, N, D, device="cuda", generator=g) for _ in range(3))
    q = (q * (1 + 20 * (torch.rand_like(q) > 0.99))).bfloat16()      # 1 % of the entries 20 times larger
    k, v = k.bfloat16(), v.bfloat16()
    bias = torch.randn(1, 4, N, N, device="cuda", generator=g).bfloat16()
    mask = torch.ones(1, 4, N, device="cuda")
    mask[0, 1] = 0               # a row with every key masked: uniform weights, finite output
    mask[0, 2, 1:] = 0           # a row with one key left
    out, _ = torch.ops.df3.attention_fwd(q, k, v, bias, mask, D**-0.5, False)
    assert bool(torch.isfinite(out).all())
    ref = _attention_reference(q, k, v, bias, mask, D**-0.5)
    live = [0, 2, 3]   # the fully masked row has no defined answer once |logit| exceeds the fp32 spacing at 1e9 (64):
    _close(out[:, live], ref[:, live], atol=4e-2, rtol=3e-2)   # every statement rounds the logits away differently
    assert float(out[0, 1].abs().max()) <= float(v[0, 1].float().abs().max()) + 1e-2   # still a convex combination of V
    _close(out[0, 2], v[0, 2, :, :1, :].expand_as(out[0, 2]), atol=1e-2, rtol=1e-2)   # the one visible key wins outright


@pytest.mark.parametrize("magnitude", [1e-2, 1.0, 20.0, 200.0])
def test_fused_epilogues_on_saturating_and_heavy_tailed_inputs(nat, magnitude):
    """Gated, SwiGLU and sigmoid-gate epilogues when the pre-activations saturate the sigmoid (|x| up to hundreds) and
    carry outliers: per-element agreement with the fp32 statement on bf16-rounded operands."""
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(1500, 128, device="cuda", generator=g)
    x = (x * (1 + 10 * (torch.rand_like(x) > 0.995))).bfloat16()
    w = (magnitude * 0.1 * torch.randn(256, 128, device="cuda", generator=g)).bfloat16()
    xf, wf = x.float(), w.float()
    gate, proj = xf @ wf[:128].t(), xf @ wf[128:].t()
    scale = proj.abs().max().item()
    got = torch.ops.df3.gemm(x, w, None, None, None, 1, False)
    _close(got, torch.sigmoid(gate) * proj, atol=1e-2 * max(scale, 1e-3), rtol=2e-2)
    got = torch.ops.df3.gemm(x, w, None, None, None, 2, False)
    want = torch.nn.functional.silu(gate) * proj
    _close(got, want, atol=1e-2 * max(want.abs().max().item(), 1e-3), rtol=2e-2)
    other = torch.randn(1500, 128, device="cuda", generator=g).bfloat16()
    got = torch.ops.df3.gemm(x, w[:128].contiguous(), None, None, other, 3, False)
    _close(got, torch.sigmoid(gate) * other.float(), atol=2e-2, rtol=2e-2)
    assert torch.ops.df3.gemm_status() == 0


def test_model_path_with_a_ragged_token_count(nat):
    """101 tokens (not a multiple of 8, 16 or 128) through a bf16 Pairformer block, forward and backward: finite, and
    close to the fp32 PyTorch statement of the same block."""
    from deepfold3_dev_b200.models.evoformer import PairFormerBlock
    from tests.helpers import wake_zero_init

    torch.manual_seed(1)
    block = PairFormerBlock(128, 384).cuda().eval()
    wake_zero_init(block)
    N = 101
    pair = torch.randn(1, N, N, 128, device="cuda", requires_grad=True)
    single = torch.randn(1, N, 384, device="cuda", requires_grad=True)
    seq_mask = torch.ones(1, N, device="cuda")
    seq_mask[0, -4:] = 0
    pair_mask = seq_mask[:, :, None] * seq_mask[:, None, :]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        p, s = block(pair, single, pair_mask, seq_mask)
    (p.float().square().mean() + s.float().square().mean()).backward()
    assert bool(torch.isfinite(p).all()) and bool(torch.isfinite(pair.grad).all()) and bool(torch.isfinite(single.grad).all())
    import os

    os.environ["DF3_DISABLE_OPS"] = "gemm,matmul,gated_dual_linear,transition,pair_bias_attention,linear_planes,sigmoid_gate_mul,layer_norm,plane_layer_norm"
    try:
        with torch.no_grad():
            p32, s32 = block(pair.detach(), single.detach(), pair_mask, seq_mask)
    finally:
        del os.environ["DF3_DISABLE_OPS"]
    err = (p.float() - p32).pow(2).mean().sqrt() / p32.pow(2).mean().sqrt()
    assert float(err) < 2e-2, float(err)
