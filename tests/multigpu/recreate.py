"""Destroy a communicator, create a new one on a new server (the library's form of recovery)
and run the fused GEMM -> reduce_scatter on it: the new group's delivery counters start from
zero, and so must the number of calls the kernel expects them to have seen."""
import os

import torch
from common import ROOT  # noqa: F401  (puts the repository on sys.path)

import megray_b200 as mr
from megray_b200.ops import gemm_error_flag
from megray_b200.parallel.tensor_parallel import TensorParallelOps

rank = int(os.environ["RANK"])
n = int(os.environ["WORLD_SIZE"])
local = int(os.environ.get("LOCAL_RANK", rank))
torch.cuda.set_device(local)
dev = torch.device("cuda", local)
base_port = int(os.environ.get("MASTER_PORT", "29641")) + 1

T, d, fl = 1024 * n, 512, 768
Ts = T // n
g = torch.Generator(device=dev).manual_seed(11)
h = (torch.randn(T, fl, device=dev, generator=g) * 0.5).to(torch.bfloat16)
w = (torch.randn(d, fl, device=dev, generator=g) * 0.05).to(torch.bfloat16)
want = n * (h.float() @ w.float().t())[rank * Ts:(rank + 1) * Ts]

for generation in range(3):
    port = base_port + 2 * generation
    server = mr.Server(n, port) if rank == 0 else None
    comm = mr.Communicator(n, rank, "nvl").init("127.0.0.1", port)
    tp = TensorParallelOps(comm, T, d, fused=True)
    assert tp.fused
    out = torch.empty(Ts, d, dtype=torch.bfloat16, device=dev)
    for rep in range(generation + 2):  # a different number of calls per generation
        out.zero_()
        tp.gemm_rs(h, w, None, out)
        torch.cuda.synchronize()
        err = float((out.float() - want).abs().max()) / float(want.abs().max())
        assert err < 3e-2, (generation, rep, err)
        assert int(gemm_error_flag(dev).item()) == 0 and comm.status == 0
    # an all-reduce on the same group, then tear everything down
    t = torch.full((1000,), float(rank + 1), device=dev)
    o = torch.empty_like(t)
    comm.all_reduce(t, o)
    torch.cuda.synchronize()
    assert float(o[0]) == n * (n + 1) / 2
    del tp
    comm.close()
    if server is not None:
        server.close()
print(f"RANK_OK {rank}", flush=True)
