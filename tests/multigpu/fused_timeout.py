"""Device-side wait limit of a fused GEMM -> reduce_scatter call, tested without faulting or
hanging a GPU: rank 1 skips the call on the host, so the tiles of rank 0's own rows wait for
partial tiles that never arrive; after the limit the kernel records MEGRAY_TIMEOUT in the
communicator's status word, frees its tensor memory and returns.  The process then checks that the
communicator refuses further fused calls and that the GPU still runs kernels."""
import time

import torch
from common import setup

from megray_b200.parallel.tensor_parallel import TensorParallelOps

rank, n, dev, comm, server = setup()
T, d, fl = 512 * n, 512, 512
Ts = T // n
g = torch.Generator(device=dev).manual_seed(3)
h = (torch.randn(T, fl, device=dev, generator=g) * 0.5).to(torch.bfloat16)
w = (torch.randn(d, fl, device=dev, generator=g) * 0.05).to(torch.bfloat16)
tp = TensorParallelOps(comm, T, d, fused=True)
assert tp.fused
out = torch.empty(Ts, d, dtype=torch.bfloat16, device=dev)
tp.gemm_rs(h, w, None, out)  # a healthy call first
torch.cuda.synchronize()
want = n * (h.float() @ w.float().t())[rank * Ts:(rank + 1) * Ts]
assert float((out.float() - want).abs().max()) / float(want.abs().max()) < 3e-2
assert comm.status == 0

comm.set_device_timeout_ms(300)
if rank == 0:
    t0 = time.time()
    tp.gemm_rs(h, w, None, out)   # rank 1 never launches this one
    torch.cuda.synchronize()      # returns: the kernel gave up by itself
    took = time.time() - t0
    assert 0.2 < took < 8.0, took
    assert comm.status == 12, comm.status     # MEGRAY_TIMEOUT, recorded by the GEMM kernel
    try:
        tp.gemm_rs(h, w, None, out)
        raise AssertionError("a failed communicator must refuse further fused calls")
    except RuntimeError as e:
        assert "12" in str(e), e
    y = torch.ones(1 << 20, device=dev).sum().item()  # the context is intact
    assert y == float(1 << 20)
else:
    time.sleep(2.0)  # stays alive, with nothing in flight, while rank 0's wait runs out
    assert comm.status == 0
print(f"RANK_OK {rank}", flush=True)
# each rank tears down on its own: the group is broken, so no collective shutdown is attempted
comm.abort()
comm.close()
