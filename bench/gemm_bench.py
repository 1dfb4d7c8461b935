#!/usr/bin/env python
"""Times the library's tcgen05 bf16 GEMM against torch.matmul (cuBLAS) on one GPU.

    python bench/gemm_bench.py                     # the TP-MLP shapes, all operand layouts
    python bench/gemm_bench.py --m 8192 --n 8192 --k 8192 --layout nt --iters 1 --no-cublas
                                                   # a single small case (for an ncu capture)

CUDA events on the launching stream, best of --iters after --warmup launches; operands
are larger than L2 for the default shapes.  Reports TFLOP/s and the fraction of the measured
cuBLAS peak in MEASURED_PEAKS.json when that file is present.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from megray_b200.ops import EPI_SWIGLU, gemm  # noqa: E402


def time_it(fn, warmup, iters):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    best = 1e30
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn", "tt", "swiglu"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--epilogue", type=int, default=0, help="0 = per-lane stores, 5 = row segments through smem")
    ap.add_argument("--variant", type=int, default=0, help="0 = automatic (CTA pair), 1 = single-CTA tile")
    a = ap.parse_args()
    peak = None
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops")
    if a.m:
        cases = [(a.layout, a.m, a.n, a.k)]
    else:
        T, d, f = 32768, 8192, 28672
        cases = [("swiglu", T, f, d), ("nt", T, d, f), ("nn", T, f, d), ("nn", T, d, 2 * f),
                 ("tt", d, f, T), ("tt", 2 * f, d, T), ("nt", 8192, 8192, 8192)]
    dev = "cuda"
    for layout, M, N, K in cases:
        a_mn = layout in ("tn", "tt")
        b_mn = layout in ("nn", "tt")
        A = torch.randn((K, M) if a_mn else (M, K), device=dev).to(torch.bfloat16)
        if layout == "swiglu":
            B = torch.randn(2 * N, K, device=dev).to(torch.bfloat16) * 0.02
            out = torch.empty(M, 2 * N, device=dev, dtype=torch.bfloat16)
            out2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: gemm(A, B, out, epilogue=EPI_SWIGLU, out2=out2, n=N, variant=a.variant)  # noqa: E731
            flops = 2.0 * M * 2 * N * K
        else:
            B = torch.randn((K, N) if b_mn else (N, K), device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda: gemm(A, B, out, a_mn=a_mn, b_mn=b_mn, variant=a.variant, epilogue=a.epilogue)  # noqa: E731
            flops = 2.0 * M * N * K
        t = time_it(fn, a.warmup, a.iters)
        line = f"{layout:7s} M={M:6d} N={N:6d} K={K:6d}  ours {t:8.3f} ms {flops / t / 1e9:7.1f} TFLOP/s"
        if peak:
            line += f" ({flops / t / 1e9 / peak:.2f} of measured {peak:.0f})"
        if not a.no_cublas:
            Af = A.t() if a_mn else A
            Bf = B if b_mn else B.t()
            if layout == "swiglu":
                ref_out = torch.empty(M, 2 * N, device=dev, dtype=torch.bfloat16)
            else:
                ref_out = out
            t2 = time_it(lambda: torch.matmul(Af, Bf, out=ref_out), a.warmup, a.iters)
            line += f" | cuBLAS {t2:8.3f} ms {flops / t2 / 1e9:7.1f} TFLOP/s | ours/cuBLAS {t2 / t:.3f}"
        print(line, flush=True)
        del A, B, out


if __name__ == "__main__":
    main()
