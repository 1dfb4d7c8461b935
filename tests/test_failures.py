"""Failure detection on the host side (no GPU is faulted, trapped or hung): a rank that never
arrives, an aborted group, use before init, and a server that goes away."""
import threading
import time

import numpy as np
import pytest

import megray_b200 as mr
from helpers import run_threads


def _group(n, timeout_ms):
    server = mr.Server(n)

    def make(rank):
        c = mr.Communicator(n, rank, "shm").init("127.0.0.1", server.port)
        c.set_host_timeout_ms(timeout_ms)
        return c

    return server, run_threads(n, make)


def test_withheld_rank_makes_the_others_time_out():
    server, comms = _group(3, 300)

    def body(rank):
        if rank == 2:
            return "absent"  # never enters the collective
        x = np.ones(8, np.float32)
        t0 = time.time()
        try:
            comms[rank].all_reduce(x, x.copy())
            return "ok"
        except mr.MegRayError as e:
            return e.status, time.time() - t0

    res = run_threads(3, body)
    for r in (0, 1):
        status, took = res[r]
        assert status in (12, 13) and took < 5  # TIMEOUT, or ABORTED after the first one gave up
    assert comms[0].status != 0 and comms[0].stats()["timeouts"] >= 0
    # the group stays failed: later calls return at once
    with pytest.raises(mr.MegRayError):
        comms[0].host_barrier()
    for c in comms:
        c.close()
    server.close()


def test_abort_releases_a_waiting_rank():
    server, comms = _group(2, 10_000)
    out = {}

    def waiter():
        try:
            comms[0].host_barrier()
            out["r"] = "ok"
        except mr.MegRayError as e:
            out["r"] = e.status

    t = threading.Thread(target=waiter, daemon=True)
    t.start()
    time.sleep(0.2)
    comms[1].abort()
    t.join(5)
    assert out["r"] == 13  # ABORTED
    assert comms[1].status == 13
    for c in comms:
        c.close()
    server.close()


def test_use_before_init_is_an_error_not_a_crash():
    c = mr.Communicator(2, 0, "shm")
    x = np.ones(4, np.float32)
    with pytest.raises(mr.MegRayError) as e:
        c.all_reduce(x, x.copy())
    assert e.value.status == 7  # INVALID_USAGE


def test_recovery_is_a_new_group_on_a_new_server():
    server, comms = _group(2, 200)
    with pytest.raises(mr.MegRayError):
        comms[0].host_barrier()  # rank 1 does not come: the group is dead afterwards
    for c in comms:
        c.close()
    server.close()
    server, comms = _group(2, 5000)  # elastic recovery = destroy and re-init

    def body(rank):
        x = np.full(4, rank + 1.0, np.float32)
        out = np.empty_like(x)
        comms[rank].all_reduce(x, out)
        return out[0]

    assert run_threads(2, body) == [3.0, 3.0]
    for c in comms:
        c.close()
    server.close()


def test_server_stop_fails_pending_clients():
    server = mr.Server(2)
    clients = run_threads(2, lambda r: _connect(server, r))
    res = {}

    def wait():
        try:
            clients[0].barrier()
            res["r"] = "ok"
        except mr.MegRayError as e:
            res["r"] = e.status

    t = threading.Thread(target=wait, daemon=True)
    t.start()
    time.sleep(0.1)
    server.stop()
    t.join(5)
    assert res["r"] in (1, 12)
    server.close()


def _connect(server, rank):
    c = mr.Client(2, rank, 3000)
    c.connect("127.0.0.1", server.port)
    return c
