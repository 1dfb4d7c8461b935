"""Host backend (MEGRAY_SHM) with CPU ranks and no GPU.

* the CPU plumbing configuration: 2 ranks on localhost through the TCP rendezvous, float32
  buffers of 1024 elements drawn uniform[-1,1] from seed 0 per rank; all_reduce SUM/MAX/MIN,
  all_gather, reduce_scatter, broadcast(root 0) and send/recv against numpy, rtol 1e-6;
* the reference's operation tests (test/test_opr.cpp:63-552): 3 ranks, 10 float32 elements,
  closed-form inputs (i+1)*(j+1), every operation, root 1 for the rooted ones;
* what the reference leaves out: every dtype, odd sizes, multi-piece messages, ranks as
  processes, grouped crossing sends."""
import numpy as np
import pytest

import megray_b200 as mr
from helpers import run_processes, with_group

NP_OPS = {"sum": np.add, "max": np.maximum, "min": np.minimum}


def rank_data(rank, n=1024, dtype=np.float32, seed=0):
    # "seed 0 per rank": each rank owns an independent stream derived from the base seed
    rng = np.random.default_rng([seed, rank])
    if np.issubdtype(dtype, np.floating):
        return rng.uniform(-1, 1, n).astype(dtype)
    return rng.integers(-100 if np.issubdtype(dtype, np.signedinteger) else 0, 100, n).astype(dtype)


def reduce_ref(arrays, op):
    out = arrays[0].copy()
    for a in arrays[1:]:
        out = NP_OPS[op](out, a).astype(arrays[0].dtype)
    return out


# ---------------------------------------------------------------------- plumbing configuration

@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_two_ranks_all_reduce(op):
    def body(comm, rank):
        x = rank_data(rank)
        out = np.empty_like(x)
        comm.all_reduce(x, out, op)
        return out

    res = with_group(2, "shm", body)
    want = reduce_ref([rank_data(0), rank_data(1)], op)
    for out in res:
        np.testing.assert_allclose(out, want, rtol=1e-6)


def test_two_ranks_all_gather_reduce_scatter_broadcast_sendrecv():
    def body(comm, rank):
        x = rank_data(rank)
        ag = np.empty(2 * x.size, np.float32)
        comm.all_gather(x, ag)
        rs = np.empty(x.size // 2, np.float32)
        comm.reduce_scatter(x, rs, "sum")
        bc = np.empty_like(x)
        comm.broadcast(x if rank == 0 else None, bc, 0)
        pr = np.empty_like(x)
        if rank == 0:
            comm.send(x, 1)
            comm.recv(pr, 1)
        else:
            comm.recv(pr, 0)
            comm.send(x, 0)
        return ag, rs, bc, pr

    res = with_group(2, "shm", body)
    x0, x1 = rank_data(0), rank_data(1)
    for rank, (ag, rs, bc, pr) in enumerate(res):
        np.testing.assert_allclose(ag, np.concatenate([x0, x1]), rtol=1e-6)
        np.testing.assert_allclose(rs, (x0 + x1)[rank * 512:(rank + 1) * 512], rtol=1e-6)
        np.testing.assert_allclose(bc, x0, rtol=1e-6)
        np.testing.assert_allclose(pr, x1 if rank == 0 else x0, rtol=1e-6)


# ---------------------------------------------------------------------- reference operation tests

N, LEN, ROOT = 3, 10, 1


def closed_form(i, n=LEN):
    return np.array([(i + 1) * (j + 1) for j in range(n)], dtype=np.float32)


def test_send_recv_chars():
    msg = np.frombuffer(b"test_message", dtype=np.uint8).copy()

    def body(comm, rank):
        if rank == 0:
            comm.send(msg, 1, dtype=mr.CHAR)
            return None
        out = np.zeros_like(msg)
        comm.recv(out, 0, dtype=mr.CHAR)
        return out.tobytes()

    assert with_group(2, "shm", body)[1] == b"test_message"


def test_scatter_gather_root1():
    def body(comm, rank):
        full = np.concatenate([closed_form(i) for i in range(N)]) if rank == ROOT else None
        part = np.empty(LEN, np.float32)
        comm.scatter(full, part, ROOT)  # non-root send buffer is null, as in the reference test
        back = np.empty(N * LEN, np.float32) if rank == ROOT else None
        comm.gather(part, back, ROOT)   # non-root recv buffer is null
        return part, back

    res = with_group(N, "shm", body)
    for rank, (part, back) in enumerate(res):
        np.testing.assert_array_equal(part, closed_form(rank))
        if rank == ROOT:
            np.testing.assert_array_equal(back, np.concatenate([closed_form(i) for i in range(N)]))


def test_all_to_all():
    def body(comm, rank):
        send = np.array([100 * rank + 10 * (k // 2) + k % 2 for k in range(2 * N)], dtype=np.float32)
        recv = np.empty_like(send)
        comm.all_to_all(send, recv)
        return recv

    res = with_group(N, "shm", body)
    for rank, recv in enumerate(res):
        want = np.array([100 * (k // 2) + 10 * rank + k % 2 for k in range(2 * N)], dtype=np.float32)
        np.testing.assert_array_equal(recv, want)  # chunk r of recv came from rank r


def test_all_gather():
    res = with_group(N, "shm", lambda c, r: _ag(c, r))
    want = np.concatenate([closed_form(i) for i in range(N)])
    for out in res:
        np.testing.assert_array_equal(out, want)


def _ag(comm, rank):
    out = np.empty(N * LEN, np.float32)
    comm.all_gather(closed_form(rank), out)
    return out


@pytest.mark.parametrize("op", ["sum", "max", "min"])
def test_all_reduce_reduce_scatter_reduce(op):
    def body(comm, rank):
        x = closed_form(rank, N * LEN)
        ar = np.empty_like(x)
        comm.all_reduce(x, ar, op)
        rs = np.empty(LEN, np.float32)
        comm.reduce_scatter(x, rs, op)
        rd = np.full(N * LEN, -1, np.float32)
        comm.reduce(x, rd if rank == ROOT else None, ROOT, op)
        return ar, rs, rd

    res = with_group(N, "shm", body)
    want = reduce_ref([closed_form(i, N * LEN) for i in range(N)], op)
    for rank, (ar, rs, rd) in enumerate(res):
        np.testing.assert_array_equal(ar, want)
        np.testing.assert_array_equal(rs, want[rank * LEN:(rank + 1) * LEN])
        if rank == ROOT:
            np.testing.assert_array_equal(rd, want)


def test_broadcast_root1_distinct_buffers():
    def body(comm, rank):
        send = closed_form(rank)
        recv = np.zeros(LEN, np.float32)
        comm.broadcast(send, recv, ROOT)
        return recv

    for out in with_group(N, "shm", body):
        np.testing.assert_array_equal(out, closed_form(ROOT))  # the root's recv buffer too


# ---------------------------------------------------------------------- beyond the reference

ALL_DTYPES = [np.int8, np.uint8, np.int32, np.uint32, np.int64, np.uint64, np.float16, np.float32, np.float64]


@pytest.mark.parametrize("dtype", ALL_DTYPES)
def test_all_reduce_every_dtype_odd_length(dtype):
    n, length = 4, 1031

    def body(comm, rank):
        x = rank_data(rank, length, dtype)
        out = np.empty_like(x)
        comm.all_reduce(x, out, "sum")
        mx = np.empty_like(x)
        comm.all_reduce(x, mx, "max")
        return out, mx

    res = with_group(n, "shm", body)
    xs = [rank_data(r, length, dtype) for r in range(n)]
    if dtype == np.float16:
        acc = sum(x.astype(np.float32) for x in xs)
        want = acc.astype(np.float16)
    else:
        with np.errstate(over="ignore"):
            want = reduce_ref(xs, "sum")
    for out, mx in res:
        if np.issubdtype(dtype, np.floating):
            np.testing.assert_allclose(out.astype(np.float64), want.astype(np.float64), rtol=2e-3, atol=1e-6)
        else:
            np.testing.assert_array_equal(out, want)
        np.testing.assert_array_equal(mx, reduce_ref(xs, "max"))


def test_messages_larger_than_the_staging_slots(monkeypatch):
    monkeypatch.setenv("MEGRAY_HOST_SLOT_KB", "64")  # force many pieces
    n, length = 3, 100_003

    def body(comm, rank):
        x = rank_data(rank, length)
        ar = np.empty_like(x)
        comm.all_reduce(x, ar)
        ag = np.empty(n * length, np.float32)
        comm.all_gather(x, ag)
        a2a_in = rank_data(rank, n * 5001)
        a2a = np.empty_like(a2a_in)
        comm.all_to_all(a2a_in, a2a)
        rs = np.empty(length // n, np.float32)
        comm.reduce_scatter(x[: (length // n) * n], rs)
        return ar, ag, a2a, rs

    res = with_group(n, "shm", body)
    xs = [rank_data(r, length) for r in range(n)]
    total = xs[0] + xs[1] + xs[2]
    a2a_ins = [rank_data(r, n * 5001) for r in range(n)]
    m = length // n
    for rank, (ar, ag, a2a, rs) in enumerate(res):
        np.testing.assert_allclose(ar, total, rtol=1e-6)
        np.testing.assert_array_equal(ag, np.concatenate(xs))
        want = np.concatenate([a2a_ins[q][rank * 5001:(rank + 1) * 5001] for q in range(n)])
        np.testing.assert_array_equal(a2a, want)
        np.testing.assert_allclose(rs, total[rank * m:(rank + 1) * m], rtol=1e-6)


def test_grouped_crossing_sends_do_not_block():
    big = 3_000_000  # bytes: far more than one mailbox holds

    def body(comm, rank):
        other = 1 - rank
        x = np.full(big, rank + 1, np.uint8)
        out = np.zeros(big, np.uint8)
        comm.group_start()
        comm.send(x, other)   # both ranks send first: only grouping makes this safe
        comm.recv(out, other)
        comm.group_end()
        return int(out[0]), int(out[-1])

    assert with_group(2, "shm", body) == [(2, 2), (1, 1)]


def test_stats_and_backend():
    def body(comm, rank):
        x = np.ones(16, np.float32)
        comm.all_reduce(x, x.copy())
        return comm.stats(), comm.backend, comm.status

    for st, backend, status in with_group(2, "shm", body):
        assert backend == mr.SHM and status == 0
        assert st["calls"] == 1 and st["bytes"] == 64


def test_nvl_only_calls_are_refused_by_other_backends():
    """Buffer registration and the symmetric heap belong to the NVL backend; the host backend
    answers MEGRAY_INVALID_USAGE instead of pretending."""
    import ctypes as C

    from megray_b200 import _lib

    def body(comm, rank):
        lib = _lib.load()
        x = np.ones(16, np.float32)
        rc_reg = lib.megray_nvl_register(comm._h, C.c_void_p(x.ctypes.data), x.nbytes)
        rc_dereg = lib.megray_nvl_deregister(comm._h, C.c_void_p(x.ctypes.data))
        ptr = lib.megray_nvl_alloc(comm._h, 1024, None)
        return rc_reg, rc_dereg, ptr

    for rc_reg, rc_dereg, ptr in with_group(2, "shm", body):
        assert rc_reg == 7 and rc_dereg == 7 and not ptr


def test_unbuilt_backends_throw_unknown_backend():
    for b in ("ucx", "rccl"):
        with pytest.raises(mr.MegRayError):
            mr.Communicator(2, 0, b)


def _proc_rank(rank, nranks, port):
    import numpy as np
    import megray_b200 as mr

    comm = mr.Communicator(nranks, rank, "shm").init("127.0.0.1", port)
    x = np.full(5000, rank + 1, np.float64)
    out = np.empty_like(x)
    comm.all_reduce(x, out)
    ag = np.empty(nranks * 3, np.int32)
    comm.all_gather(np.full(3, rank, np.int32), ag)
    comm.close()
    return float(out[0]), ag.tolist()


def test_ranks_as_processes_share_a_posix_shm_region():
    n = 3
    server = mr.Server(n)
    res = run_processes(n, _proc_rank, n, server.port)
    server.close()
    for total, ag in res:
        assert total == 6.0
        assert ag == [0, 0, 0, 1, 1, 1, 2, 2, 2]


def test_python_ops_refuse_buffers_that_break_the_length_contract():
    """The native calls trust the length contracts of include/megray/communicator.h; the Python
    layer checks them (and the dtypes) first, so a short buffer raises instead of being overrun."""
    import pytest

    port = mr.get_free_port()
    server = mr.Server(1, port)
    comm = mr.Communicator(1, 0, "host").init("127.0.0.1", port)
    a4, a8 = np.zeros(4, np.float32), np.zeros(8, np.float32)
    i4 = np.zeros(4, np.int32)
    with pytest.raises(ValueError):
        comm.all_reduce(a8, a4)
    with pytest.raises(ValueError):
        comm.all_reduce(a4, i4)
    with pytest.raises(ValueError):
        comm.all_gather(a4, a8)          # nranks == 1: recv must hold exactly send.numel
    with pytest.raises(ValueError):
        comm.reduce_scatter(a8, a4)
    with pytest.raises(ValueError):
        comm.all_to_all(a4, a8)
    with pytest.raises(ValueError):
        comm.broadcast(a8, a4, 0)
    with pytest.raises(ValueError):
        comm.gather(a4, a8, 0)
    with pytest.raises(ValueError):
        comm.scatter(a8, a4, 0)
    with pytest.raises(ValueError):
        comm.reduce(a4, a8, 0)
    comm.all_reduce(a4, a4.copy())       # a call that keeps the contract still works
    comm.close()
    server.close()
