"""The host (shared-memory) backend driven with CUDA tensors: staged through pinned host memory,
reduced on the CPU, and stream-ordered: a call enqueues its copies, a hand-over to the
communicator's worker thread and a stream wait, and returns without waiting for the GPU
(the semantics of the reference's shared-memory all_reduce, src/shm/all_reduce.cpp:88-124).
Two ranks as threads of this process, both on GPU 0 (the backend launches no kernels of its own,
so nothing on the device waits for anything else on it)."""
import threading
import time

import numpy as np
import pytest
import torch

import megray_b200 as mr

pytestmark = pytest.mark.gpu


def test_cuda_tensors_through_the_host_backend_without_blocking_the_caller():
    n = 2
    port = mr.get_free_port()
    server = mr.Server(n, port)
    results, errors = {}, []

    def rank_main(r):
        try:
            torch.cuda.set_device(0)
            comm = mr.Communicator(n, r, "host").init("127.0.0.1", port)
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                x = torch.full((1 << 20,), float(r + 1), device="cuda")
                y = torch.zeros_like(x)
                g = torch.zeros(n * 1000, device="cuda")
                comm.all_reduce(x, y, "sum", stream=stream)           # warm-up: buffers, worker thread
                stream.synchronize()
                # keep the stream busy for a while, then issue the collective: the call must
                # return while the earlier work is still running
                big = torch.randn(8192, 8192, device="cuda")
                started = torch.cuda.Event()
                for _ in range(40):
                    big = big @ big * 1e-4
                started.record(stream)
                t0 = time.perf_counter()
                comm.all_reduce(x, y, "max", stream=stream)
                comm.all_gather(x[:1000], g, stream=stream)
                host_ms = (time.perf_counter() - t0) * 1000.0
                still_running = not started.query()
                stream.synchronize()
                results[r] = (host_ms, still_running, float(y[0]), float(y[-1]), g[:1000].unique().tolist(),
                              g[1000:].unique().tolist(), comm.status)
            comm.close()
        except Exception as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = [threading.Thread(target=rank_main, args=(r,)) for r in range(n)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(120)
    server.close()
    assert not errors, errors
    for r in range(n):
        host_ms, still_running, y0, y1, g0, g1, status = results[r]
        assert status == 0
        assert y0 == float(n) and y1 == float(n)            # max over ranks of (r + 1)
        assert g0 == [1.0] and g1 == [2.0]
        assert still_running, "the matmuls had finished before the call returned: nothing to conclude"
        assert host_ms < 50.0, f"the call blocked the host for {host_ms:.1f} ms"


def test_host_tensors_still_work_after_cuda_tensors():
    """Host-context calls run on the caller's thread: they first let the worker finish."""
    port = mr.get_free_port()
    server = mr.Server(1, port)
    comm = mr.Communicator(1, 0, "host").init("127.0.0.1", port)
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    y = torch.zeros_like(x)
    comm.all_reduce(x, y)
    a = np.arange(16, dtype=np.float32)
    b = np.zeros_like(a)
    comm.all_reduce(a, b)
    torch.cuda.synchronize()
    assert torch.equal(x, y) and np.array_equal(a, b)
    comm.close()
    server.close()
