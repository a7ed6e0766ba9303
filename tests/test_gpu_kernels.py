"""sm_100a kernels against the fp32 PyTorch statement of the same op (``ops/reference.py``)."""

import pytest
import torch

from deepfold3_dev_b200 import ops
from deepfold3_dev_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module", autouse=True)
def _native():
    from deepfold3_dev_b200.ops import native

    native.require()


@pytest.mark.parametrize("C", [16, 64, 128, 267, 384, 768, 831])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("affine", [True, False])
def test_layer_norm_forward_backward(C, dtype, affine):
    torch.manual_seed(0)
    x = (torch.randn(3, 37, C, device=DEV) * 3 + 1).to(dtype).requires_grad_(True)
    w = torch.randn(C, device=DEV, requires_grad=True) if affine else None
    b = torch.randn(C, device=DEV, requires_grad=True) if affine else None
    y = ops.layer_norm(x, w, b, 1e-5)
    assert ops.census()["layer_norm:sm100"] > 0
    x32 = x.detach().float().requires_grad_(True)
    w32 = w.detach().clone().requires_grad_(True) if affine else None
    b32 = b.detach().clone().requires_grad_(True) if affine else None
    y32 = ref.layer_norm(x32, w32, b32, 1e-5)
    tol = dict(atol=4e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=2e-5, rtol=1e-5)
    torch.testing.assert_close(y.float(), y32, **tol)
    g = torch.randn_like(y32)
    y.backward(g.to(dtype))
    y32.backward(g)
    gtol = dict(atol=8e-2, rtol=5e-2) if dtype == torch.bfloat16 else dict(atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(x.grad.float(), x32.grad, **gtol)
    if affine:
        wtol = dict(atol=0.5, rtol=5e-2) if dtype == torch.bfloat16 else dict(atol=1e-3, rtol=1e-4)
        torch.testing.assert_close(w.grad, w32.grad, **wtol)
        torch.testing.assert_close(b.grad, b32.grad, **wtol)


@pytest.mark.parametrize("C", [64, 130, 768, 1024])
@pytest.mark.parametrize("x_dtype", [torch.float32, torch.bfloat16])
def test_adaptive_layer_norm_and_gated_residual(C, x_dtype):
    """``sigmoid(s) * LN(x) + t`` and ``a + sigmoid(z) * u`` in one kernel each way against the fp32 statement: values,
    and the gradients of every operand (the residual stream is fp32 under autocast, the conditioning tensors bf16)."""
    torch.manual_seed(C)
    shape = (2, 5, 37, C)
    x = (torch.randn(*shape, device=DEV) * 2 + 0.5).to(x_dtype).requires_grad_(True)
    s = torch.randn(*shape, device=DEV).bfloat16().requires_grad_(True)
    t = torch.randn(*shape, device=DEV).bfloat16().requires_grad_(True)
    ops.census(reset=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        y = ops.ada_norm(x, s, t, 1e-5)
    assert ops.census().get("ada_norm:sm100", 0) == 1 and y.dtype == torch.bfloat16
    w = torch.randn(*shape, device=DEV)
    (y.float() * w).sum().backward()
    x32, s32, t32 = (v.detach().float().requires_grad_(True) for v in (x, s, t))
    want = torch.sigmoid(s32) * torch.nn.functional.layer_norm(x32, (C,), None, None, 1e-5) + t32
    (want * w.bfloat16().float()).sum().backward()  # the incoming gradient reaches the kernel rounded to bf16
    assert (y.float() - want).abs().max().item() < 0.04
    for got, ref_t, name in ((x.grad, x32.grad, "x"), (s.grad, s32.grad, "s"), (t.grad, t32.grad, "t")):
        scale = ref_t.abs().max().item()
        assert got.dtype == (x_dtype if name == "x" else torch.bfloat16)
        assert (got.float() - ref_t).abs().max().item() < 0.02 * scale + 1e-3, name

    a = torch.randn(*shape, device=DEV).to(x_dtype).requires_grad_(True)
    z = torch.randn(*shape, device=DEV).bfloat16().requires_grad_(True)
    u = torch.randn(*shape, device=DEV).bfloat16().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        r = ops.gated_residual(a, z, u)
    assert ops.census().get("gated_residual:sm100", 0) == 1 and r.dtype == x_dtype
    (r.float() * w).sum().backward()
    a32, z32, u32 = (v.detach().float().requires_grad_(True) for v in (a, z, u))
    want = a32 + torch.sigmoid(z32) * u32
    (want * (w.to(x_dtype).float())).sum().backward()
    assert (r.float() - want).abs().max().item() < (1e-5 if x_dtype == torch.float32 else 0.04)
    for got, ref_t, name in ((a.grad, a32.grad, "a"), (z.grad, z32.grad, "z"), (u.grad, u32.grad, "u")):
        assert (got.float() - ref_t).abs().max().item() < 0.02 * ref_t.abs().max().item() + 1e-3, name
    # shapes that do not match (a conditioning tensor shared by the samples) take the PyTorch statement
    ops.census(reset=True)
    with torch.autocast("cuda", dtype=torch.bfloat16):
        ops.ada_norm(x.detach(), s.detach()[:, :1], t.detach()[:, :1])
        ops.gated_residual(a.detach(), z.detach()[:, :1], u.detach())
    assert ops.census().get("ada_norm:torch", 0) == 1 and ops.census().get("gated_residual:torch", 0) == 1


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_swiglu(dtype):
    torch.manual_seed(1)
    x = torch.randn(5, 33, 2 * 96, device=DEV).to(dtype).requires_grad_(True)
    y = ops.swiglu(x)
    x32 = x.detach().float().requires_grad_(True)
    y32 = ref.swiglu(x32)
    tol = dict(atol=3e-2, rtol=2e-2) if dtype == torch.bfloat16 else dict(atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(y.float(), y32, **tol)
    g = torch.randn_like(y32)
    y.backward(g.to(dtype))
    y32.backward(g)
    torch.testing.assert_close(x.grad.float(), x32.grad, **(dict(atol=6e-2, rtol=3e-2) if dtype == torch.bfloat16 else tol))


@pytest.mark.parametrize("share_dim", [-3, -2])
def test_dropout_add_mask_is_shared_and_unbiased(share_dim):
    torch.manual_seed(2)
    res = torch.zeros(2, 40, 48, 32, device=DEV)
    x = torch.ones(2, 40, 48, 32, device=DEV, requires_grad=True)
    out = ops.dropout_add(res, x, 0.25, True, share_dim)
    m = out.detach().clone()  # the scaled mask itself since x == 1 and the residual is 0
    vals = torch.unique(m).tolist()
    assert all(v == 0.0 or abs(v - 1 / 0.75) < 1e-6 for v in vals)
    ref_slice = m.select(share_dim, 0).unsqueeze(share_dim)
    assert torch.equal(m, ref_slice.expand_as(m))  # identical along the shared axis
    keep = float((m > 0).float().mean())
    assert abs(keep - 0.75) < 0.03
    out.sum().backward()
    torch.testing.assert_close(x.grad, m)  # backward regenerates the same mask
    out2 = ops.dropout_add(res, x.detach(), 0.25, True, share_dim)
    assert not torch.equal(out2, out.detach())  # a new call draws a new mask
    # residual and values: same seed, bf16 (vector kernel) against the mask applied by hand
    from deepfold3_dev_b200.ops import autograd_ops

    r16, x16 = torch.randn(2, 40, 48, 32, device=DEV).bfloat16(), torch.randn(2, 40, 48, 32, device=DEV).bfloat16()
    mask = autograd_ops.dropout_add(torch.zeros_like(x16), torch.ones_like(x16), 0.25, share_dim, seed=77).float()
    got = autograd_ops.dropout_add(r16, x16, 0.25, share_dim, seed=77).float()
    torch.testing.assert_close(got, (r16.float() + x16.float() * mask).bfloat16().float(), atol=2e-2, rtol=2e-2)


def test_dropout_add_eval_is_plain_add():
    a, b = torch.randn(3, 4, 5, device=DEV), torch.randn(3, 4, 5, device=DEV)
    torch.testing.assert_close(ops.dropout_add(a, b, 0.25, False, -3), a + b)


def test_flat_adamw_kernel_matches_reference_math():
    from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW

    def build(dev):
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(64, 96), torch.nn.LayerNorm(96), torch.nn.Linear(96, 8)).to(dev)

    gpu, cpu = build(DEV), build("cpu")
    og = FlatAdamW(gpu, lr=1e-2, weight_decay=0.1, ema_decay=0.9)
    oc = FlatAdamW(cpu, lr=1e-2, weight_decay=0.1, ema_decay=0.9)
    x = torch.randn(16, 64)
    for step in range(3):
        cpu(x).pow(2).sum().backward()
        # the same gradients on both sides: the test is about the update rule, and Adam's normalisation would blow up
        # the last-bit differences between a GPU and a CPU backward pass
        og.flat_grad.copy_(oc.flat_grad.to(DEV))
        og.step(grad_scale=torch.tensor(0.5, device=DEV))
        oc.step(grad_scale=0.5)
        og.zero_grad()
        oc.zero_grad()
    torch.testing.assert_close(og.flat_param.cpu(), oc.flat_param, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(og.shadow.cpu(), oc.shadow, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(og.exp_avg_sq.cpu(), oc.exp_avg_sq, atol=1e-8, rtol=1e-5)


def test_peer_flag_wait_runs_out_and_reports_status():
    """A wait for a flag that nothing sets ends after its poll limit with a status code; the context stays usable.

    One GPU plays rank 0 of a world of two whose second rank never runs: its control block is plain local memory.
    """
    from deepfold3_dev_b200.ops import native

    native.require()
    n = 4096
    grads = [torch.randn(n, device=DEV), torch.randn(n, device=DEV)]
    ctrls = [torch.zeros(256, device=DEV), torch.zeros(256, device=DEV)]
    ctrls[0][0] = 1.0
    ctrls[1][0] = 1.0
    scratch = torch.zeros(4, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    before = grads[0].clone()
    norm = torch.ops.df3.peer_allreduce_mean(grads[0], [g.data_ptr() for g in grads], [c.data_ptr() for c in ctrls], scratch,
                                             status, 0, 2, 1, 20000)  # fmt: skip
    torch.cuda.synchronize()
    assert int(status.item()) == 4  # kTimeoutPeerFlag
    assert torch.isnan(norm)
    assert torch.equal(grads[0], before)  # the entry wait ran out: no gradient was read or written
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0  # the device still answers


def _fused_step_setup(ema_decay=0.9, weight_decay=0.1):
    from deepfold3_dev_b200.parallel.dist import DistInfo
    from deepfold3_dev_b200.parallel.peer_reduce import PeerReducer
    from deepfold3_dev_b200.training.flat_optimizer import FlatAdamW

    def build(dev):
        torch.manual_seed(5)
        return torch.nn.Sequential(torch.nn.Linear(64, 200), torch.nn.LayerNorm(200), torch.nn.Linear(200, 33)).to(dev)

    gpu, cpu = build(DEV), build("cpu")
    og = FlatAdamW(gpu, lr=1e-2, weight_decay=weight_decay, ema_decay=ema_decay)
    oc = FlatAdamW(cpu, lr=1e-2, weight_decay=weight_decay, ema_decay=ema_decay)
    peer = PeerReducer(DistInfo(device=torch.device(DEV)), og)
    return gpu, cpu, og, oc, peer


def _launch_fused(og, peer, loss_flag=0.0, clip=0.0, thr=0.0):
    step = og.step_count + 1
    b1, b2 = og.param_groups[0]["betas"]
    one = torch.ones((), device=DEV)
    peer.fused_step(og, coef=one, loss_flag=torch.tensor(loss_flag, device=DEV), local_norm=torch.zeros((), device=DEV),
                    lr=og.param_groups[0]["lr"], betas=(b1, b2), eps=og.param_groups[0]["eps"], bc1=1 - b1**step, bc2=1 - b2**step,
                    ema=og.shadow, ema_w=1 - og.ema_decay, clip_norm=clip, skip_threshold=thr, per_rank_clip=False)  # fmt: skip
    res = peer.read_result()
    if res["advanced"]:
        og.step_count = step
    return res


def test_fused_optimizer_step_matches_flat_adamw():
    """One cooperative kernel (entry, reduce, norm, consensus, AdamW, EMA, bf16 mirror, gradient zeroing) on a world of
    one against the CPU statement of clip + AdamW + EMA lerp, three steps."""
    gpu, cpu, og, oc, peer = _fused_step_setup()
    x = torch.randn(16, 64)
    for _ in range(3):
        cpu(x).pow(2).sum().backward()
        og.flat_grad.copy_(oc.flat_grad)  # the same gradient bits on both sides: only the update is under test
        norm = oc.grad_norm(True)
        scale = min(1.0, 0.5 / (float(norm) + 1e-6))
        res = _launch_fused(og, peer, clip=0.5)
        assert res["advanced"] and res["reason"] is None
        assert abs(res["norm"] - float(norm)) < 1e-4 * float(norm) and abs(res["scale"] - scale) < 1e-5
        oc.step(grad_scale=scale)
        oc.zero_grad()
        assert float(og.flat_grad.abs().max()) == 0.0  # zeroed by the kernel for the next window
    torch.testing.assert_close(og.flat_param.cpu(), oc.flat_param, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(og.shadow.cpu(), oc.shadow, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(og.exp_avg.cpu(), oc.exp_avg, atol=1e-7, rtol=1e-5)
    torch.testing.assert_close(og.exp_avg_sq.cpu(), oc.exp_avg_sq, atol=1e-8, rtol=1e-5)
    torch.testing.assert_close(og.flat_param_bf16.float().cpu(), oc.flat_param.bfloat16().float(), atol=1e-2, rtol=1e-2)
    peer.check()


@pytest.mark.parametrize("case", ["loss", "grad", "outlier"])
def test_fused_optimizer_step_skips_on_device(case):
    """The skip decision is taken inside the kernel: parameters, moments and EMA stay untouched, gradients are cleared."""
    gpu, cpu, og, oc, peer = _fused_step_setup()
    gpu(torch.randn(16, 64, device=DEV)).pow(2).sum().backward()
    if case == "grad":
        og.flat_grad[7] = float("nan")
    before = [t.clone() for t in (og.flat_param, og.exp_avg, og.exp_avg_sq, og.shadow)]
    res = _launch_fused(og, peer, loss_flag=1.0 if case == "loss" else 0.0, thr=1e-3 if case == "outlier" else 0.0)
    assert not res["advanced"] and res["reason"] == ("loss" if case == "loss" else "grad")
    for a, b in zip(before, (og.flat_param, og.exp_avg, og.exp_avg_sq, og.shadow)):
        assert torch.equal(a, b)
    assert float(og.flat_grad.nan_to_num().abs().max()) == 0.0


def test_fused_step_entry_wait_runs_out_and_reports_status():
    """Rank 0 of a world of two whose second rank never arrives: the entry wait ends after its poll limit, the kernel
    records the status and leaves without reading or writing any gradient or parameter; the context stays usable."""
    from deepfold3_dev_b200.ops import native

    native.require()
    n = 4096
    grads = [torch.randn(n, device=DEV), torch.randn(n, device=DEV)]
    ctrls = [torch.zeros(256, device=DEV), torch.zeros(256, device=DEV)]
    p, m, v, ema, decay = (torch.randn(n, device=DEV) for _ in range(5))
    before = [t.clone() for t in (grads[0], p, m, v, ema)]
    scratch, status = torch.zeros(4, device=DEV), torch.zeros(1, dtype=torch.int32, device=DEV)
    result = torch.full((36,), -1.0, device=DEV)
    torch.ops.df3.peer_fused_step(grads[0], [g.data_ptr() for g in grads], [c.data_ptr() for c in ctrls], scratch, status, result,
                                  p, m, v, ema, decay, None, 0, 2, 1, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.05, 0.001, 1.0, 0.0, False, 20000)  # fmt: skip
    torch.cuda.synchronize()
    assert int(status.item()) == 4  # kTimeoutPeerFlag
    assert float(result[0]) == 0.0 and float(result[1]) == 3.0
    for a, b in zip(before, (grads[0], p, m, v, ema)):
        assert torch.equal(a, b)
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0  # the device still answers
