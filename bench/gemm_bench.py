#!/usr/bin/env python
"""Times the library's tcgen05 bf16 GEMM against torch.matmul (cuBLAS) on one GPU.

    python bench/gemm_bench.py                     # the TP-MLP shapes, all operand layouts
    python bench/gemm_bench.py --m 8192 --n 8192 --k 8192 --layout nt --iters 1 --no-cublas
                                                   # a single small case (for an ncu capture)

CUDA events on the launching stream around each launch.  All candidates of a case (each
variant asked for, then cuBLAS) are launched in turn, --iters rounds after --warmup rounds, and
the median per candidate is reported, so that a drift of the power-capped clock during the case
hits every candidate alike.  Operands are larger than L2 for the default shapes.  Reports TFLOP/s and the fraction of the measured
cuBLAS peak in MEASURED_PEAKS.json when that file is present.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from megray_b200.ops import EPI_DSWIGLU, EPI_SWIGLU, gemm, gemm_split_k  # noqa: E402


def time_round_robin(fns, warmup, iters):
    """Median milliseconds per candidate, candidates launched in turn."""
    for _ in range(warmup):
        for fn in fns:
            fn()
    torch.cuda.synchronize()
    times = [[] for _ in fns]
    for _ in range(iters):
        for i, fn in enumerate(fns):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times[i].append(e0.elapsed_time(e1))
    return [sorted(t)[len(t) // 2] for t in times]


def time_sustained(fn, seconds, index=0):
    """Runs `fn` back to back for about `seconds` under the clock sampler.  Returns milliseconds per
    launch (CUDA events around the whole loop) and the sampler's record: at the power cap the
    clock the kernel settles at tells how much energy one launch costs."""
    from megray_b200.utils.clocks import ClockSampler

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    n = max(5, int(seconds * 1000.0 / max(e0.elapsed_time(e1), 1e-3)))
    sampler = ClockSampler(index).start()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    rec = sampler.stop()
    return e0.elapsed_time(e1) / n, rec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--m", type=int)
    ap.add_argument("--n", type=int)
    ap.add_argument("--k", type=int)
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn", "tt", "swiglu", "dswiglu"])
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--epilogue", type=int, default=0, help="0 = per-lane stores, 5 = row segments through smem")
    ap.add_argument("--variant", type=int, default=0, help="0 = automatic, 1 = single-CTA 128x256 tile, 2 = CTA-pair 256x256 tile, 3 = CTA-pair 512x256 tile")
    ap.add_argument("--split-k", default="", help="comma-separated K-range counts to time as extra candidates "
                                                    "(plain layouts; 1 = no split)")
    ap.add_argument("--sustain", type=float, default=0.0,
                    help="also run every candidate back to back for this many seconds and report its time, "
                         "median SM MHz, maximum power and time x MHz (energy per launch at the power cap)")
    ap.add_argument("--variants", default="", help="comma-separated variants to time one after the other on each case")
    a = ap.parse_args()
    variants = [int(v) for v in a.variants.split(",")] if a.variants else [a.variant]
    peak = None
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops")
    if a.m:
        cases = [(a.layout, a.m, a.n, a.k)]
    else:
        T, d, f = 32768, 8192, 28672
        cases = [("swiglu", T, f, d), ("nt", T, d, f), ("dswiglu", T, f, d), ("nn", T, f, d), ("nn", T, d, 2 * f),
                 ("tt", d, f, T), ("tt", 2 * f, d, T), ("nt", 8192, 8192, 8192)]
    dev = "cuda"
    for layout, M, N, K in cases:
        a_mn = layout in ("tn", "tt")
        b_mn = layout in ("nn", "tt", "dswiglu")
        A = torch.randn((K, M) if a_mn else (M, K), device=dev).to(torch.bfloat16)
        if layout == "swiglu":
            B = torch.randn(2 * N, K, device=dev).to(torch.bfloat16) * 0.02
            out = torch.empty(M, 2 * N, device=dev, dtype=torch.bfloat16)
            out2 = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda v: gemm(A, B, out, epilogue=EPI_SWIGLU, out2=out2, n=N, variant=v)  # noqa: E731
            flops = 2.0 * M * 2 * N * K
        elif layout == "dswiglu":
            # backward of the SwiGLU projection: dH = dY @ W_down (NN), epilogue turns it into
            # [dG | dU] with the saved [G | U]
            B = torch.randn(K, N, device=dev).to(torch.bfloat16) * 0.02
            aux = torch.randn(M, 2 * N, device=dev).to(torch.bfloat16)
            out = torch.empty(M, 2 * N, device=dev, dtype=torch.bfloat16)
            fn = lambda v: gemm(A, B, out, b_mn=True, epilogue=EPI_DSWIGLU, aux=aux, n=N, variant=v)  # noqa: E731
            flops = 2.0 * M * N * K
        else:
            B = torch.randn((K, N) if b_mn else (N, K), device=dev).to(torch.bfloat16)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            fn = lambda v: gemm(A, B, out, a_mn=a_mn, b_mn=b_mn, variant=v, epilogue=a.epilogue)  # noqa: E731
            flops = 2.0 * M * N * K
        cands = [(lambda v=v: fn(v)) for v in variants]
        splits = [int(x) for x in a.split_k.split(",")] if a.split_k and layout in ("nt", "nn", "tn", "tt") else []
        for sk in splits:
            ws = torch.empty(sk * M, N, device=dev, dtype=torch.float32)
            cands.append(lambda sk=sk, ws=ws: gemm_split_k(A, B, out, sk, ws, a_mn=a_mn, b_mn=b_mn))
        if not a.no_cublas:
            Af = A.t() if a_mn else A
            Bf = B if b_mn else B.t()
            ref_out = torch.empty(M, 2 * N, device=dev, dtype=torch.bfloat16) if layout == "swiglu" else (
                torch.empty(M, N, device=dev, dtype=torch.bfloat16) if layout == "dswiglu" else out)
            cands.append(lambda: torch.matmul(Af, Bf, out=ref_out))
        ts = time_round_robin(cands, a.warmup, a.iters)
        line = f"{layout:7s} M={M:6d} N={N:6d} K={K:6d} "
        for v, t in zip(variants, ts):
            line += f" ours{'' if len(variants) == 1 else f'[v{v}]'} {t:8.3f} ms {flops / t / 1e9:7.1f} TFLOP/s"
            if peak:
                line += f" ({flops / t / 1e9 / peak:.2f} of measured {peak:.0f})"
        for sk, t in zip(splits, ts[len(variants):]):
            line += f" split-k[{sk}] {t:8.3f} ms {flops / t / 1e9:7.1f} TFLOP/s"
        if not a.no_cublas:
            t2 = ts[-1]
            line += f" | cuBLAS {t2:8.3f} ms {flops / t2 / 1e9:7.1f} TFLOP/s | ours/cuBLAS " + \
                    "/".join(f"{t2 / t:.3f}" for t in ts[:-1])
        print(line, flush=True)
        if a.sustain > 0:
            names = [f"ours[v{v}]" for v in variants] + [f"split-k[{sk}]" for sk in splits] + \
                    ([] if a.no_cublas else ["cuBLAS"])
            for name, fn_c in zip(names, cands):
                t, rec = time_sustained(fn_c, a.sustain)
                mhz = rec.get("sm_mhz") or 0.0
                print(f"    sustained {a.sustain:.0f} s  {name:12s} {t:8.3f} ms {flops / t / 1e9:7.1f} TFLOP/s  "
                      f"median {mhz:.0f} MHz  max {rec.get('power_w_max')} W  temp {rec.get('temp_c')}  "
                      f"reasons {rec.get('reasons')}  time x MHz {t * mhz:9.1f}", flush=True)
        del A, B, out


if __name__ == "__main__":
    main()
