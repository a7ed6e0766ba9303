"""The allocation-free C entry point (``ops/csrc/no_alloc_entry.h``) against the regular LayerNorm backward op.

Collected last on purpose (file name): it must pass alone and after every other GPU test has used the device.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from deepfold3_dev_b200.ops import native

    native.require()
    lib = ctypes.CDLL(native.so_path())
    fn = lib.df3_layer_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 8 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.df3_no_alloc_last_error.restype = ctypes.c_char_p
    return lib


def _case(rows, channels, dtype, seed, with_weight=True):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, channels, device="cuda", generator=g).to(dtype)
    dy = torch.randn(rows, channels, device="cuda", generator=g).to(dtype)
    w = (torch.rand(channels, device="cuda", generator=g) + 0.5) if with_weight else None
    xf = x.float()
    mean = xf.mean(-1)
    rstd = torch.rsqrt(xf.var(-1, unbiased=False) + 1e-5)
    return x, dy, w, mean.contiguous(), rstd.contiguous()


def _run_both(lib, x, dy, w, mean, rstd):
    dx_ref, partial = torch.ops.df3.layer_norm_bwd(dy, x, w, mean, rstd, True)
    sums = partial.sum(0)
    dx = torch.full_like(x, float("nan"))
    dw = torch.full((x.shape[1],), float("nan"), device="cuda")
    db = torch.full((x.shape[1],), float("nan"), device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.df3_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr() if w is not None else None,
                                        mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                        x.shape[0], x.shape[1], int(x.dtype == torch.bfloat16), stream)  # fmt: skip
    assert rc == 0, lib.df3_no_alloc_last_error().decode()
    torch.cuda.synchronize()
    return (dx, dw, db), (dx_ref, sums[0], sums[1])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_matches_regular_entry_point_on_two_calls_in_a_row(dtype):
    lib = _lib()
    # the second call has another shape, so stale partial sums of the first would show up
    for seed, (rows, channels) in enumerate([(5000, 128), (777, 384)]):
        x, dy, w, mean, rstd = _case(rows, channels, dtype, seed)
        (dx, dw, db), (dx_ref, dw_ref, db_ref) = _run_both(lib, x, dy, w, mean, rstd)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=tol, atol=tol)
        torch.testing.assert_close(dw, dw_ref, rtol=1e-4, atol=1e-2 if dtype == torch.bfloat16 else 1e-3)
        torch.testing.assert_close(db, db_ref, rtol=1e-4, atol=1e-2 if dtype == torch.bfloat16 else 1e-3)


def test_allocates_nothing_and_rejects_oversize():
    lib = _lib()
    x, dy, w, mean, rstd = _case(1024, 256, torch.bfloat16, 7)
    _run_both(lib, x, dy, w, mean, rstd)  # first call on the device does the one-time set-up
    dx = torch.empty_like(x)
    dw = torch.empty(256, device="cuda")
    db = torch.empty(256, device="cuda")
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    stats_before = torch.cuda.memory_stats()["allocation.all.allocated"]
    rc = lib.df3_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(),
                                        dx.data_ptr(), dw.data_ptr(), db.data_ptr(), 1024, 256, 1,
                                        torch.cuda.current_stream().cuda_stream)  # fmt: skip
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.cuda.memory_stats()["allocation.all.allocated"] == stats_before
    assert torch.cuda.mem_get_info()[0] == free_before
    rc = lib.df3_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), None, mean.data_ptr(), rstd.data_ptr(),
                                        dx.data_ptr(), dw.data_ptr(), db.data_ptr(), 4, 2048, 1, None)  # fmt: skip
    assert rc == -1
    assert b"2048" in lib.df3_no_alloc_last_error()


@pytest.mark.parametrize("rows,channels", [(300, 1024), (50, 600), (37, 100)])
def test_channel_counts_up_to_the_limit_and_odd_shapes(rows, channels):
    """The widest supported row (1024 channels: the fixed scratch array is used to its end), a channel count that is
    not a multiple of the vector width, and a small odd shape."""
    lib = _lib()
    for dtype in (torch.float32, torch.bfloat16):
        x, dy, w, mean, rstd = _case(rows, channels, dtype, 11)
        (dx, dw, db), (dx_ref, dw_ref, db_ref) = _run_both(lib, x, dy, w, mean, rstd)
        tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
        torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=tol, atol=tol)
        torch.testing.assert_close(dw, dw_ref, rtol=1e-4, atol=1e-2 if dtype == torch.bfloat16 else 1e-3)
        torch.testing.assert_close(db, db_ref, rtol=1e-4, atol=1e-2 if dtype == torch.bfloat16 else 1e-3)


def test_parameter_gradients_may_be_left_out():
    """``dw`` and ``db`` null together: only ``dx`` is computed, and it equals the ``dx`` of a full call."""
    lib = _lib()
    x, dy, w, mean, rstd = _case(513, 256, torch.bfloat16, 13)
    (dx_full, _, _), _ = _run_both(lib, x, dy, w, mean, rstd)
    dx = torch.full_like(x, float("nan"))
    rc = lib.df3_layer_norm_bwd_noalloc(dy.data_ptr(), x.data_ptr(), w.data_ptr(), mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                                        None, None, x.shape[0], x.shape[1], 1, torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc == 0, lib.df3_no_alloc_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_full)
