"""Per-kernel timing of the sm_100a ops against their library / eager counterparts.

    python -m deepfold3_dev_b200.ops.microbench --op attention --iters 10
    python -m deepfold3_dev_b200.ops.microbench --op all

Each case is timed with CUDA events after three warm-up calls, a 256 MB buffer is rewritten between
timed calls so inputs do not sit in L2, and the median is printed with the achieved fraction of the
measured copy bandwidth / GEMM throughput (``MEASURED_PEAKS.json`` beside the repository root when
present). Shapes are the ones the 384-token training step runs.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from . import native, reference as ref

N = 384


def _peaks():
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d.get("hbm_gbs", 6650.0)), float(d.get("bf16_tflops", 1590.0)), "measured"
    except (OSError, ValueError):
        return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self, iters: int):
        self.iters = iters
        self.flush = torch.zeros(64 * 1024 * 1024, device="cuda")

    def __call__(self, fn) -> float:
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(self.iters):
            self.flush.add_(1)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]


def _report(name, ms, other_ms, nbytes, flops):
    gbs, tfl, kind = _peaks()
    line = f"{name:34s} {ms * 1e3:9.1f} us"
    line += f"   library/eager {other_ms * 1e3:9.1f} us" if other_ms is not None else " " * 28
    if nbytes:
        line += f"   {nbytes / ms / 1e6:7.0f} GB/s ({nbytes / ms / 1e6 / gbs:.2f} of {kind} copy)"
    if flops:
        line += f"   {flops / ms / 1e9:7.0f} TFLOP/s ({flops / ms / 1e9 / tfl:.2f} of {kind} cuBLAS)"
    print(line, flush=True)


def bench_gemm(t: Timer):
    df3 = torch.ops.df3
    rows = N * N
    x = torch.randn(rows, 128, device="cuda").bfloat16()
    w = torch.randn(128, 128, device="cuda").bfloat16() * 0.1
    w2 = torch.randn(256, 128, device="cuda").bfloat16() * 0.1
    w1 = torch.randn(1024, 128, device="cuda").bfloat16() * 0.1
    o = torch.randn(rows, 128, device="cuda").bfloat16()
    io = lambda *n: 2 * rows * sum(n)  # noqa: E731 - bf16 bytes moved for the given channel counts
    _report(f"gemm plain {rows}x128->128", t(lambda: df3.gemm(x, w, None, None, None, 0, False)), t(lambda: x @ w.t()),
            io(128, 128), 2 * rows * 128 * 128)  # fmt: skip
    _report(f"gemm gated {rows}x128->128", t(lambda: df3.gemm(x, w2, None, None, None, 1, False)),
            t(lambda: torch.sigmoid(x @ w2[:128].t()) * (x @ w2[128:].t())), io(128, 128), 2 * rows * 128 * 256)  # fmt: skip
    _report(f"gemm swiglu {rows}x128->512", t(lambda: df3.gemm(x, w1, None, None, None, 2, False)),
            t(lambda: ref.swiglu(x @ w1.t())), io(128, 512), 2 * rows * 128 * 1024)  # fmt: skip
    _report(f"gemm sigmoid-mul {rows}x128->128", t(lambda: df3.gemm(x, w, None, None, o, 3, False)),
            t(lambda: torch.sigmoid(x @ w.t()) * o), io(128, 128, 128), 2 * rows * 128 * 128)  # fmt: skip
    w3 = torch.randn(384, 128, device="cuda").bfloat16() * 0.1
    _report(f"gemm plain {rows}x128->384", t(lambda: df3.gemm(x, w3, None, None, None, 0, False)), t(lambda: x @ w3.t()),
            io(128, 384), 2 * rows * 128 * 384)  # fmt: skip
    _report(f"gemm gated planes {rows}x128->128", t(lambda: df3.gemm(x, w2, None, None, None, 1, True)),
            t(lambda: (torch.sigmoid(x @ w2[:128].t()) * (x @ w2[128:].t())).t().contiguous()), io(128, 128), 2 * rows * 128 * 256)  # fmt: skip
    _report(f"matmul dx {rows}x128 . 128x128", t(lambda: df3.matmul(o, w, False, False, False, 1)), t(lambda: o @ w),
            io(128, 128), 2 * rows * 128 * 128)  # fmt: skip
    _report(f"matmul dw ({rows}x128)^T . {rows}x128", t(lambda: df3.matmul(o, x, True, False, True, 0)), t(lambda: (o.t() @ x).float()),
            io(128, 128), 2 * rows * 128 * 128)  # fmt: skip
    pa, pb = torch.randn(128, N, N, device="cuda").bfloat16(), torch.randn(128, N, N, device="cuda").bfloat16()
    _report(f"triangle contraction out 128x{N}^3", t(lambda: df3.matmul(pa, pb, False, True, False, 1)),
            t(lambda: torch.bmm(pa, pb.transpose(1, 2))), 3 * 2 * 128 * N * N, 2 * 128 * N**3)  # fmt: skip
    _report(f"triangle contraction in 128x{N}^3", t(lambda: df3.matmul(pb, pa, True, False, False, 1)),
            t(lambda: torch.bmm(pb.transpose(1, 2), pa)), 3 * 2 * 128 * N * N, 2 * 128 * N**3)  # fmt: skip
    M = 8192
    A, B = torch.randn(M, M, device="cuda").bfloat16(), torch.randn(M, M, device="cuda").bfloat16()
    _report("gemm plain 8192^3", t(lambda: df3.gemm(A, B, None, None, None, 0, False)), t(lambda: A @ B.t()), 0, 2 * M**3)
    _report("matmul NN 8192^3", t(lambda: df3.matmul(A, B, False, False, False, 1)), t(lambda: A @ B), 0, 2 * M**3)


def bench_attention(t: Timer):
    df3 = torch.ops.df3
    for B, R, H, D, name in [(1, N, 4, 32, "triangle"), (1, 48, 16, 48, "diffusion"), (1, 1, 16, 24, "single")]:
        q, k, v = (torch.randn(B, R, H, N, D, device="cuda").bfloat16() for _ in range(3))
        bias = torch.randn(B, H, N, N, device="cuda").bfloat16()
        mask = torch.ones(B, R, N, device="cuda")
        ours = t(lambda: df3.attention_fwd(q, k, v, bias, mask, D**-0.5, True))
        eager = t(lambda: ref.pair_bias_attention(q, k, v, bias, mask, D**-0.5, False))
        _report(f"attention fwd {name}", ours, eager, 2 * 4 * B * R * H * N * D, 4 * B * R * H * N * N * D)
        out, lse, out32 = df3.attention_fwd_train(q, k, v, bias, mask, D**-0.5)
        d_out = torch.randn_like(out)
        fused = t(lambda: df3.attention_bwd(q, k, v, out32, d_out, bias, mask, lse, D**-0.5, True, 40 << 20))
        chunked = t(lambda: df3.attention_bwd(q, k, v, out, d_out, bias, mask, lse, D**-0.5, True, -(40 << 20)))
        # five products of 2 N N D per (b, r, h); the chunked form (library GEMMs + one kernel per chunk) is the comparison
        _report(f"attention bwd {name}", fused, chunked, 2 * 8 * B * R * H * N * D, 10 * B * R * H * N * N * D)


def bench_elementwise(t: Timer):
    from . import autograd_ops as ao

    x = torch.randn(1, N, N, 128, device="cuda").bfloat16()
    r = torch.randn_like(x)
    w = torch.ones(128, device="cuda")
    nb = x.numel() * 2
    planes = torch.randn(128, N * N, device="cuda").bfloat16()
    _report(f"plane_layer_norm fwd 128x{N * N}", t(lambda: torch.ops.df3.plane_layer_norm_fwd(planes, w, w, 1e-5)),
            t(lambda: torch.nn.functional.layer_norm(planes.t(), (128,), w.bfloat16(), w.bfloat16())), 2 * nb, 0)  # fmt: skip
    _report(f"layer_norm fwd {N * N}x128", t(lambda: torch.ops.df3.layer_norm_fwd(x, w, w, 1e-5)),
            t(lambda: torch.nn.functional.layer_norm(x, (128,), w.bfloat16(), w.bfloat16())), 2 * nb, 0)  # fmt: skip
    _report(f"dropout_add rows {N * N}x128", t(lambda: ao.dropout_add(r, x, 0.25, -3, seed=1)),
            t(lambda: r + torch.nn.functional.dropout(x, 0.25)), 3 * nb, 0)  # fmt: skip


def bench_streaming(t: Timer):
    """Bandwidth-bound kernels on tensors larger than L2 (768-token pair tensor, 151 MB in bf16; 92 M-element optimizer)."""
    n = 768
    x = torch.randn(n * n, 128, device="cuda").bfloat16()
    w = torch.ones(128, device="cuda")
    nb = x.numel() * 2
    y, mean, rstd = torch.ops.df3.layer_norm_fwd(x, w, w, 1e-5)
    _report("layer_norm fwd 589824x128", t(lambda: torch.ops.df3.layer_norm_fwd(x, w, w, 1e-5)),
            t(lambda: torch.nn.functional.layer_norm(x, (128,), w.bfloat16(), w.bfloat16())), 2 * nb, 0)  # fmt: skip
    _report("layer_norm bwd 589824x128", t(lambda: torch.ops.df3.layer_norm_bwd(y, x, w, mean, rstd, True)), None, 3 * nb, 0)
    planes = torch.randn(128, n * n, device="cuda").bfloat16()
    _report("plane_layer_norm fwd 128x589824", t(lambda: torch.ops.df3.plane_layer_norm_fwd(planes, w, w, 1e-5)),
            t(lambda: torch.nn.functional.layer_norm(planes.t(), (128,), w.bfloat16(), w.bfloat16())), 2 * nb, 0)  # fmt: skip
    h = torch.randn(n * n // 4, 1024, device="cuda").bfloat16()
    _report("swiglu fwd 147456x1024", t(lambda: torch.ops.df3.swiglu_fwd(h)),
            t(lambda: torch.nn.functional.silu(h[:, :512]) * h[:, 512:]), h.numel() * 3, 0)  # fmt: skip
    m = 92_000_000
    p, g, m1, m2, ema = (torch.randn(m, device="cuda") * 0.01 for _ in range(5))
    m2.abs_()
    p16 = torch.empty(m, device="cuda", dtype=torch.bfloat16)
    decay, scale = torch.zeros(m, device="cuda"), torch.ones(1, device="cuda")
    _report("adamw+ema+bf16 mirror 92M", t(lambda: torch.ops.df3.adamw_ema(p, g, m1, m2, ema, decay, scale, 1e-3, 0.9, 0.95, 1e-8,
                                                                            0.1, 0.05, 1e-3, p16)), None, m * (4 * 10 + 2), 0)  # fmt: skip


def bench_diffusion(t: Timer):
    """Element-wise kernels of the diffusion transformer at the training shape (48 samples x N tokens x 768 channels:
    the fp32 residual stream is 57 MB at N = 384, with its conditioning tensors well beyond L2), and the atom-window
    attention (N * 24 / 32 windows of 32 queries x 128 keys, 4 heads of 32, bias shared by the samples)."""
    S, C = 48, 768
    x = torch.randn(S, N, C, device="cuda")
    s, sh, dy = (torch.randn(S, N, C, device="cuda").bfloat16() for _ in range(3))
    rows_bytes = x.numel()

    def eager_ada():
        return (torch.sigmoid(s.float()) * torch.nn.functional.layer_norm(x, (C,)) + sh.float()).bfloat16()

    _report(f"ada_ln fwd {S * N}x{C}", t(lambda: torch.ops.df3.ada_ln_fwd(x, s, sh, 1e-5)), t(eager_ada), rows_bytes * (4 + 2 + 2 + 2), 0)
    _, mean, rstd = torch.ops.df3.ada_ln_fwd(x, s, sh, 1e-5)
    _report(f"ada_ln bwd {S * N}x{C}", t(lambda: torch.ops.df3.ada_ln_bwd(dy, x, s, mean, rstd)), None, rows_bytes * (2 + 4 + 2 + 4 + 2), 0)
    _report(f"gated_residual fwd {S * N}x{C}", t(lambda: torch.ops.df3.gated_residual_fwd(x, s, sh)),
            t(lambda: x + torch.sigmoid(s.float()) * sh.float()), rows_bytes * (4 + 2 + 2 + 4), 0)  # fmt: skip
    _report(f"gated_residual bwd {S * N}x{C}", t(lambda: torch.ops.df3.gated_residual_bwd(x, s, sh)), None, rows_bytes * (4 + 2 + 2 + 2 + 2), 0)

    from . import autograd_ops as ao

    W, H, Q, Kk, D = N * 24 // 32, 4, 32, 128, 32
    q = torch.randn(1, S, W, H, Q, D, device="cuda").bfloat16()
    k, v = (torch.randn(1, S, W, H, Kk, D, device="cuda").bfloat16() for _ in range(2))
    bias = torch.randn(1, 1, W, H, Q, Kk, device="cuda").bfloat16()
    if ao.window_attention_supported(q, k, v, bias):
        nbytes = 2 * (2 * q.numel() + k.numel() + v.numel() + bias.numel())
        _report(f"window attention {S}x{W} windows", t(lambda: ao.window_attention(q, k, v, bias, D**-0.5)),
                t(lambda: ref.window_attention(q, k, v, bias, D**-0.5)), nbytes, 4 * S * W * H * Q * Kk * D)  # fmt: skip


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="all", choices=["all", "gemm", "attention", "elementwise", "streaming", "diffusion"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=384, help="token count of the pair-shaped cases (384: training crop, 1024: inference)")
    args = ap.parse_args()
    global N
    N = args.tokens
    native.require()
    t = Timer(args.iters)
    if args.op in ("all", "gemm"):
        bench_gemm(t)
    if args.op in ("all", "attention"):
        bench_attention(t)
    if args.op in ("all", "elementwise"):
        bench_elementwise(t)
    if args.op in ("all", "streaming"):
        bench_streaming(t)
    if args.op in ("all", "diffusion"):
        bench_diffusion(t)
    code = torch.ops.df3.gemm_status()
    print("kernel status word:", code)
    if code != 0:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
