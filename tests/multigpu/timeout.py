"""Device-side wait limit, tested without faulting or hanging a GPU: rank 1 does not launch the
collective that rank 0 launches (a host-side skip between steps), so rank 0's kernel waits for a
flag nobody sets; after the limit it records MEGRAY_TIMEOUT in the status word and returns.  The
process then checks that the GPU still runs kernels and that the communicator reports the failure
to later calls."""
import time

import torch
from common import setup

rank, n, dev, comm, server = setup()
x = torch.ones(1024, device=dev)
out = torch.empty_like(x)
comm.all_reduce(x, out)  # a healthy call first
torch.cuda.synchronize()
assert float(out[0]) == n

comm.set_device_timeout_ms(300)
if rank == 0:
    t0 = time.time()
    comm.all_reduce(x, out)      # rank 1 never joins this one
    torch.cuda.synchronize()     # returns: the kernel gave up by itself
    took = time.time() - t0
    assert 0.2 < took < 5.0, took
    assert comm.status == 12, comm.status          # MEGRAY_TIMEOUT
    assert comm.stats()["timeouts"] >= 1
    try:
        comm.all_reduce(x, out)
        raise AssertionError("a failed communicator must refuse further calls")
    except Exception as e:  # noqa: BLE001
        assert "TIMEOUT" in str(e), e
    y = torch.ones(1 << 20, device=dev).sum().item()  # the context is intact
    assert y == float(1 << 20)
else:
    time.sleep(1.5)  # stays alive, with nothing in flight, while rank 0's wait runs out
    assert comm.status == 0
print(f"RANK_OK {rank}", flush=True)
# each rank tears down on its own: the group is broken, so no collective shutdown is attempted
comm.abort()
comm.close()
