#!/usr/bin/env python
"""Fused tensor-parallel kernels against their unfused forms and their roofline.

    torchrun --nproc-per-node N bench/tp_fused_bench.py [--tokens 32768 --d 8192 --ffn 28672]

For the all_gather -> GEMM (SwiGLU up/gate projection) and the GEMM -> reduce_scatter (down
projection) of one layer it times, per rank, on the device with CUDA events (max over ranks):
the GEMM alone on local data, the collective alone, collective + GEMM back to back, and the
fused kernel (candidates launched in turn; median over --iters rounds).  The roofline of a fused kernel is the slower of FLOPs / measured GEMM peak and
bytes over NVLink / measured link bandwidth (MEASURED_PEAKS.json and 770 GB/s per direction).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

from megray_b200.ops import EPI_SWIGLU, gemm  # noqa: E402
from megray_b200.parallel.tensor_parallel import TensorParallelOps  # noqa: E402
from megray_b200.utils import init_from_env, max_over_ranks  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--d", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--ffn-shards", type=int, default=0, help="shard the FFN as if over this many ranks (default: world)")
    a = ap.parse_args()
    os.environ.setdefault("MEGRAY_HEAP_MB", "6144")
    rank, n, dev, comm, server = init_from_env()
    assert comm is not None, "run under torchrun with at least 2 ranks"
    T, d = a.tokens, a.d
    fl = a.ffn // (a.ffn_shards or n)
    Ts = T // n
    tp = TensorParallelOps(comm, T, d, fused=True)
    bf = dict(dtype=torch.bfloat16, device=dev)
    xg = tp.full_buffer()
    xg.normal_()
    w_gu = torch.randn(2 * fl, d, **bf) * 0.02
    w_dn = torch.randn(d, fl, **bf) * 0.02
    gu = torch.empty(T, 2 * fl, **bf)
    h = torch.empty(T, fl, **bf)
    h.normal_()
    partial = torch.empty(T, d, **bf)
    out = torch.empty(Ts, d, **bf)
    peak = 1400.0
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        peak = json.load(open(pk)).get("bf16_tflops_sustained", peak)
    link = 770.0

    shard = xg[rank * Ts:(rank + 1) * Ts]

    def unfused_up():
        tp.fused = False
        tp.ag_gemm_swiglu(xg, w_gu, gu, h, fl)
        tp.fused = True

    def unfused_down():
        tp.fused = False
        tp.gemm_rs(h, w_dn, partial, out)
        tp.fused = True

    cands = {
        "gemm_up": lambda: gemm(xg, w_gu, gu, epilogue=EPI_SWIGLU, out2=h, n=fl),
        "all_gather": lambda: comm.all_gather(shard, xg),
        "ag+gemm": unfused_up,
        "ag_gemm_fused": lambda: tp.ag_gemm_swiglu(xg, w_gu, gu, h, fl),
        "gemm_down": lambda: gemm(h, w_dn, partial),
        "reduce_scatter": lambda: comm.reduce_scatter(partial, out),
        "gemm+rs": unfused_down,
        "gemm_rs_fused": lambda: tp.gemm_rs(h, w_dn, None, out),
    }
    # candidates run in turn, one timed launch each per round, so that a drift of the
    # power-capped clock hits all of them alike; median over the rounds, max over ranks
    for _ in range(2):
        for fn in cands.values():
            fn()
    times = {k: [] for k in cands}
    for _ in range(a.iters):
        for k, fn in cands.items():
            torch.cuda.synchronize()
            comm.stream_barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times[k].append(e0.elapsed_time(e1))
    res = {k: max_over_ranks(comm, sorted(v)[len(v) // 2], dev) for k, v in times.items()}
    if rank == 0:
        fl_up = 2.0 * T * 2 * fl * d
        fl_dn = 2.0 * T * d * fl
        nbytes = (n - 1) / n * T * d * 2
        roof_up = max(fl_up / peak / 1e9, nbytes / link / 1e6)
        roof_dn = max(fl_dn / peak / 1e9, nbytes / link / 1e6)
        print(f"n={n} tokens={T} d={d} ffn_local={fl}  (ms, max over ranks)")
        for k, v in res.items():
            print(f"  {k:16s} {v:8.3f}")
        print(f"  roofline up   {roof_up:8.3f} ms -> fused achieves {roof_up / res['ag_gemm_fused']:.2f} of it "
              f"(unfused {roof_up / res['ag+gemm']:.2f})")
        print(f"  roofline down {roof_dn:8.3f} ms -> fused achieves {roof_dn / res['gemm_rs_fused']:.2f} of it "
              f"(unfused {roof_dn / res['gemm+rs']:.2f})")
    torch.cuda.synchronize()
    comm.close()


if __name__ == "__main__":
    main()
