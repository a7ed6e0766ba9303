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
        gpu(x.to(DEV)).pow(2).sum().backward()
        cpu(x).pow(2).sum().backward()
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
    ctrls = [torch.zeros(128, device=DEV), torch.zeros(128, device=DEV)]
    ctrls[0][0] = 1.0
    ctrls[1][0] = 1.0
    scratch = torch.zeros(4, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    norm = torch.ops.df3.peer_allreduce_mean(grads[0], [g.data_ptr() for g in grads], [c.data_ptr() for c in ctrls], scratch,
                                             status, 0, 2, 1, 20000)  # fmt: skip
    torch.cuda.synchronize()
    assert int(status.item()) == 4  # kTimeoutPeerFlag
    assert torch.isnan(norm)
    assert float((torch.ones(8, device=DEV) * 2).sum()) == 16.0  # the device still answers
