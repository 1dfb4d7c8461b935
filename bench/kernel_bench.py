#!/usr/bin/env python
"""Times the library's memory-bound kernels on one GPU against the measured copy bandwidth:
N-way reduce (the collectives' arithmetic), fused add+RMSNorm forward / backward, fused SGD,
squared-error loss, MoE dispatch and combine (all experts local).  Inputs are larger than L2;
CUDA events, best of --iters after --warmup.  `--only NAME --iters 1 --warmup 1` gives a small
single-kernel run for an ncu capture.

    python bench/kernel_bench.py [--only reduce_n|rmsnorm|rmsnorm_bwd|sgd|mse|moe_dispatch|moe_combine]
"""
import argparse
import ctypes as C
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import megray_b200 as mr  # noqa: E402
from megray_b200 import _lib  # noqa: E402
from megray_b200.ops import add_rmsnorm, mse_loss_grad, rmsnorm_bwd, sgd_step  # noqa: E402
from megray_b200.parallel.expert_parallel import ExpertParallelOps  # noqa: E402


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
    ap.add_argument("--only", default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--rows", type=int, default=32768)
    ap.add_argument("--cols", type=int, default=8192)
    a = ap.parse_args()
    lib = _lib.load()
    peak = None
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("hbm_gbs")
    dev = "cuda"
    R, Ccols = a.rows, a.cols
    bf = dict(dtype=torch.bfloat16, device=dev)
    st = lambda: C.c_void_p(torch.cuda.current_stream().cuda_stream)  # noqa: E731
    cases = {}

    def case(name):
        def deco(f):
            cases[name] = f
            return f
        return deco

    @case("reduce_n")
    def _():
        n = 4
        xs = [torch.randn(R * Ccols // 2, device=dev).to(torch.bfloat16) for _ in range(n)]
        out = torch.empty_like(xs[0])
        ptrs = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
        fn = lambda: lib.megray_reduce_n(ptrs, n, out.data_ptr(), out.numel(), mr.BFLOAT16, mr.BFLOAT16, mr.SUM,  # noqa: E731
                                         C.c_float(1.0 / n), st())
        return fn, (n + 1) * out.numel() * 2

    @case("rmsnorm")
    def _():
        x, y = torch.randn(R, Ccols, **bf), torch.randn(R, Ccols, **bf)
        xo, no = torch.empty_like(x), torch.empty_like(x)
        inv = torch.empty(R, device=dev)
        return (lambda: add_rmsnorm(x, y, xo, no, inv)), 4 * x.numel() * 2

    @case("rmsnorm_bwd")
    def _():
        dn, n_, dres = torch.randn(R, Ccols, **bf), torch.randn(R, Ccols, **bf), torch.randn(R, Ccols, **bf)
        dx = torch.empty_like(dn)
        inv = torch.rand(R, device=dev)
        return (lambda: rmsnorm_bwd(dn, n_, inv, dres, dx)), 4 * dn.numel() * 2

    @case("sgd")
    def _():
        w, g = torch.randn(R * Ccols, **bf), torch.randn(R * Ccols, **bf)
        return (lambda: sgd_step(w, g, 1e-4)), 3 * w.numel() * 2

    @case("mse")
    def _():
        y = torch.randn(R, Ccols, **bf)
        dy = torch.empty_like(y)
        return (lambda: mse_loss_grad(y, None, None, dy)), 2 * y.numel() * 2

    def moe_setup():
        T, H, E = 16384, 4096, 64
        ep = ExpertParallelOps(None, T, H, E, 1.25)
        logits = torch.randn(T, E, device=dev)
        x = torch.randn(T, H, **bf)
        ep.route(logits)
        ep.plan()
        buf = ep.exchange_buffer()
        ep.dispatch(x, buf, first=True)
        return ep, x, buf, T, H

    @case("moe_dispatch")
    def _():
        ep, x, buf, T, H = moe_setup()
        return (lambda: ep.dispatch(x, buf, first=False)), (T + 2 * T) * H * 2

    @case("moe_combine")
    def _():
        ep, x, buf, T, H = moe_setup()
        out = torch.empty_like(x)
        return (lambda: ep.combine(out, buf, weights=True)), (2 * T + T) * H * 2

    for name, make in cases.items():
        if a.only and a.only != name:
            continue
        fn, nbytes = make()
        t = time_it(fn, a.warmup, a.iters)
        gbs = nbytes / t / 1e6
        line = f"{name:14s} {t * 1000:9.1f} us  {gbs:8.1f} GB/s"
        if peak:
            line += f"  ({gbs / peak:.2f} of measured copy {peak:.0f} GB/s)"
        print(line, flush=True)


if __name__ == "__main__":
    main()
