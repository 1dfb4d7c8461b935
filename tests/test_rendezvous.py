"""Rendezvous server/client: the cases of the reference's test/test_server_client.cpp:20-216
(host ip, free port, connect, barrier ordering, broadcast from rank 1, allgather, a mixed
request sequence) plus the failure paths the reference cannot test: connect deadline,
size mismatch, a rank that never joins a round, a rank that leaves."""
import struct
import threading
import time

import pytest

import megray_b200 as mr
from helpers import run_threads

N = 3


def test_get_host_ip_is_non_loopback_ipv4_or_none():
    ip = mr.get_host_ip()
    if ip is not None:
        assert len(ip) >= 7 and ip.count(".") == 3 and not ip.startswith("127.")


def test_get_free_port():
    assert mr.get_free_port() > 0


def _clients(server, n=N, timeout_ms=None):
    def connect(rank):
        c = mr.Client(n, rank, timeout_ms)
        c.connect("127.0.0.1", server.port)
        return c

    return run_threads(n, connect)


def test_connect_and_barrier_orders_ranks():
    server = mr.Server(N)
    clients = _clients(server)
    counter = {"v": 0}
    lock = threading.Lock()

    def body(rank):
        time.sleep(0.05 * rank)  # staggered arrival, as in the reference test
        with lock:
            counter["v"] += 1
        clients[rank].barrier()
        return counter["v"]

    seen = run_threads(N, body)
    assert seen == [N] * N  # nobody left the barrier before everyone had arrived
    assert server.requests_served == 1
    for c in clients:
        c.close()
    server.close()


def test_broadcast_from_rank_1():
    server = mr.Server(N)
    clients = _clients(server)
    payload = b"0123456789"

    def body(rank):
        return clients[rank].broadcast(payload if rank == 1 else b"", len(payload), 1)

    assert run_threads(N, body) == [payload] * N
    server.close()


def test_allgather_is_rank_major():
    server = mr.Server(N)
    clients = _clients(server)

    def body(rank):
        return clients[rank].allgather(struct.pack("ii", rank, rank * rank))

    want = b"".join(struct.pack("ii", r, r * r) for r in range(N))
    assert run_threads(N, body) == [want] * N
    server.close()


def test_mixed_sequence_keeps_the_state_machine_in_step():
    server = mr.Server(N)
    clients = _clients(server)

    def body(rank):
        c = clients[rank]
        out = []
        c.barrier()
        out.append(c.broadcast(b"abcd" if rank == 0 else b"", 4, 0))
        out.append(c.allgather(bytes([rank])))
        c.barrier()
        out.append(c.broadcast(b"xy" if rank == 2 else b"", 2, 2))
        return out

    res = run_threads(N, body)
    assert res == [[b"abcd", bytes(range(N)), b"xy"]] * N
    assert server.requests_served == 5
    server.close()


def test_single_rank_group():
    server = mr.Server(1)
    c = mr.Client(1, 0)
    c.connect("127.0.0.1", server.port)
    c.barrier()
    assert c.allgather(b"zz") == b"zz"  # the reference server reads an unset length here
    assert c.broadcast(b"q", 1, 0) == b"q"
    server.close()


def test_free_function_server_serves_until_rank0_leaves():
    port = mr.get_free_port()
    mr.create_server(2, port)

    def body(rank):
        c = mr.Client(2, rank)
        c.connect("127.0.0.1", port)
        c.barrier()
        c.close()
        return True

    assert run_threads(2, body) == [True, True]


def test_connect_gives_up_when_there_is_no_server(monkeypatch):
    monkeypatch.setenv("MEGRAY_CONNECT_TIMEOUT_MS", "300")
    # options are read once per process: the Client constructor reads the global copy, so
    # set the deadline through a fresh process-wide parse is not possible; use a child instead
    import subprocess, sys, os

    code = (
        "import megray_b200 as mr, time\n"
        "c = mr.Client(2, 0)\n"
        "t = time.time()\n"
        "try:\n"
        "    c.connect('127.0.0.1', %d)\n"
        "    print('connected?')\n"
        "except mr.MegRayError as e:\n"
        "    print('status', e.status, 'after', round(time.time() - t, 1))\n"
    ) % mr.get_free_port()
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=root,
                         env=dict(os.environ, MEGRAY_CONNECT_TIMEOUT_MS="300", MEGRAY_LOG_LEVEL="3"), timeout=60)
    assert "status 12" in out.stdout, out.stdout + out.stderr  # MEGRAY_TIMEOUT


def test_size_mismatch_ends_the_service_with_an_error():
    server = mr.Server(2)
    clients = _clients(server, 2, timeout_ms=3000)

    def body(rank):
        try:
            clients[rank].allgather(b"x" * (4 if rank == 0 else 8))
            return "ok"
        except mr.MegRayError as e:
            return e.status

    res = run_threads(2, body)
    assert all(r != "ok" for r in res)
    deadline = time.time() + 5
    while server.running and time.time() < deadline:
        time.sleep(0.01)
    assert not server.running and server.status == 6  # INVALID_ARGUMENT
    server.close()


def test_rank_that_never_joins_a_round_times_the_others_out():
    server = mr.Server(2)
    clients = _clients(server, 2, timeout_ms=400)
    t0 = time.time()
    with pytest.raises(mr.MegRayError) as e:
        clients[0].barrier()  # rank 1 never calls barrier
    assert e.value.status in (12, 1)  # TIMEOUT (or SYS_ERROR if the server gave up first)
    assert time.time() - t0 < 5
    server.close()


def test_departure_of_a_rank_between_rounds_is_survived_until_the_next_request():
    server = mr.Server(2)
    clients = _clients(server, 2, timeout_ms=1000)
    run_threads(2, lambda r: clients[r].barrier())
    clients[1].close()  # rank 1 leaves cleanly between rounds
    time.sleep(0.1)
    assert server.running
    with pytest.raises(mr.MegRayError):
        clients[0].barrier()  # a request of an incomplete group cannot be served
    server.close()


def test_duplicate_rank_is_refused():
    server = mr.Server(2)
    a = mr.Client(2, 0, 500)
    results = {}

    def first():
        try:
            a.connect("127.0.0.1", server.port)
            results["a"] = "ok"
        except mr.MegRayError as e:
            results["a"] = e.status

    t = threading.Thread(target=first, daemon=True)
    t.start()
    time.sleep(0.1)
    b = mr.Client(2, 0, 500)
    with pytest.raises(mr.MegRayError):
        b.connect("127.0.0.1", server.port)  # rank 0 is already taken
    c = mr.Client(2, 1, 500)
    c.connect("127.0.0.1", server.port)
    t.join(5)
    assert results["a"] == "ok"
    server.close()
