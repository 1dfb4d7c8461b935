"""Rank harnesses for the tests: ranks as threads of this process (the way the reference's
gtest suite runs its ranks, reference test/test_base.h:25-62) or as spawned processes."""
import multiprocessing as mp
import threading
import traceback

import megray_b200 as mr


def run_threads(nranks, fn, *args, timeout=60):
    """fn(rank, *args) on one thread per rank; returns the list of results, re-raises failures."""
    results = [None] * nranks
    errors = []

    def body(r):
        try:
            results[r] = fn(r, *args)
        except BaseException as e:  # noqa: BLE001
            errors.append((r, e, traceback.format_exc()))

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(nranks)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout)
        assert not t.is_alive(), "a rank thread is stuck"
    if errors:
        r, e, tb = errors[0]
        raise AssertionError(f"rank {r} failed: {e}\n{tb}")
    return results


def with_group(nranks, backend, body, *args, timeout=60):
    """Start a server, give every rank thread an initialised communicator, run body(comm, rank, *args)."""
    server = mr.Server(nranks)

    def fn(rank):
        comm = mr.Communicator(nranks, rank, backend).init("127.0.0.1", server.port)
        try:
            return body(comm, rank, *args)
        finally:
            comm.close()

    try:
        return run_threads(nranks, fn, timeout=timeout)
    finally:
        server.close()


def _proc_entry(target, rank, args, queue):
    try:
        queue.put((rank, "ok", target(rank, *args)))
    except BaseException as e:  # noqa: BLE001
        queue.put((rank, "error", f"{e}\n{traceback.format_exc()}"))


def run_processes(nranks, target, *args, timeout=120):
    """target(rank, *args) in one spawned process per rank (target must be importable)."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    procs = [ctx.Process(target=_proc_entry, args=(target, r, args, queue)) for r in range(nranks)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(nranks):
            rank, kind, val = queue.get(timeout=timeout)
            assert kind == "ok", f"rank {rank} failed: {val}"
            out[rank] = val
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    return [out[r] for r in range(nranks)]
