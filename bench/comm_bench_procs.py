#!/usr/bin/env python
"""Collective bandwidth with one PROCESS per GPU on ordinary torch tensors: the shape in which
MegEngine drives MegRay.  (build/megray_bench runs the ranks as threads of one process, as the
reference's test/performance.cpp does.)  Under torchrun:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29750 bench/comm_bench_procs.py --backend nvl --sizes 1M,64M,1G

``--backend nvl`` is the native backend (the two buffers are registered once, so every peer has
them mapped and calls of any size take the single-pass kernels; with ``--no-register`` allocations
up to 64 MiB are still exported and mapped on first use, larger calls take the staged kernels), ``--backend nccl`` this library's wrapper around NCCL, i.e. the calls the
reference's NCCL backend makes (src/nccl/communicator.cpp:170-228).  Device-timed with CUDA
events, max over ranks; prints the JSON lines of build/megray_bench (bench/sweep_table.py reads
both).  ``bytes`` is the per-rank unit as in that tool: the whole message for all_reduce /
broadcast / reduce, one rank's share for the others.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import megray_b200 as mr  # noqa: E402

OPS = ["all_reduce", "reduce_scatter", "all_gather", "all_to_all", "broadcast", "reduce", "gather", "scatter"]


def parse_size(s):
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    return int(s[:-1]) * mult[s[-1]] if s[-1] in mult else int(s)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nvl")
    ap.add_argument("--ops", default=",".join(OPS))
    ap.add_argument("--sizes", default="64K,1M,16M,256M")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no-register", action="store_true",
                    help="nvl: leave the two buffers unregistered (calls above the automatic-export limit, 64 MiB "
                         "per buffer, then take the staged kernels)")
    a = ap.parse_args()
    rank, n = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    port = int(os.environ.get("MASTER_PORT", "29750")) + 7
    server = mr.Server(n, port) if rank == 0 else None
    comm = mr.Communicator(n, rank, a.backend).init("127.0.0.1", port)
    sizes = [parse_size(s) for s in a.sizes.split(",")]
    cap = max(sizes) // 4
    src = torch.full((cap * n,), float(rank + 1), device=dev)
    dst = torch.zeros(cap * n, device=dev)
    tmax = torch.zeros(1, device=dev)
    tall = torch.zeros(n, device=dev)
    if a.backend == "nvl" and not a.no_register:
        # one call per buffer, as a framework does for its communication buffers: every peer maps them
        assert comm.register(src) and comm.register(dst)
    for _ in range(20):  # clocks up, links trained, first-call work done
        comm.all_reduce(src[:4096], dst[:4096])
    torch.cuda.synchronize()
    for op in a.ops.split(","):
        for size in sizes:
            m = size // 4  # float32 elements of the unit
            calls = {
                "all_reduce": lambda: comm.all_reduce(src[:m], dst[:m]),
                "reduce_scatter": lambda: comm.reduce_scatter(src[:m * n], dst[:m]),
                "all_gather": lambda: comm.all_gather(src[:m], dst[:m * n]),
                "all_to_all": lambda: comm.all_to_all(src[:m * n], dst[:m * n]),
                "broadcast": lambda: comm.broadcast(src[:m], dst[:m], 0),
                "reduce": lambda: comm.reduce(src[:m], dst[:m], 0),
                "gather": lambda: comm.gather(src[:m], dst[:m * n], 0),
                "scatter": lambda: comm.scatter(src[:m * n], dst[:m], 0),
            }
            call = calls[op]
            for _ in range(a.warmup):
                call()
            comm.stream_barrier() if a.backend == "nvl" else torch.cuda.synchronize()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(a.iters):
                call()
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1000.0 / a.iters
            tmax[0] = us
            comm.all_gather(tmax, tall)
            torch.cuda.synchronize()
            us = float(tall.max())
            if rank == 0:
                factor = {"all_reduce": 2.0 * (n - 1) / n, "broadcast": 1.0, "reduce": 1.0}.get(op, float(n - 1))
                print(json.dumps({"backend": a.backend + "-procs", "op": op, "dtype": "float32",
                                  "reduce": "sum" if op in ("all_reduce", "reduce_scatter", "reduce") else "-",
                                  "bytes": size, "time_us": round(us, 2), "busbw_gbs": round(size * factor / us / 1e3, 2),
                                  "algo": "-", "ok": True, "nranks": n}), flush=True)
    st = comm.stats()
    if rank == 0 and a.backend == "nvl":
        sys.stderr.write(f"stats: {st}\n")
    comm.close()
    if server is not None:
        server.close()


if __name__ == "__main__":
    main()
