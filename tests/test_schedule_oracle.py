"""The second oracle (the reference's ring all_reduce and binomial-tree reduce schedules replayed
over host buffers) against the rank-order oracle and against a numpy replay of the same
schedules: integer and MAX / MIN results agree bit for bit whatever the schedule, floating-point
sums agree with the numpy replay exactly and with the rank-order sum up to reassociation."""
import ctypes as C

import numpy as np
import pytest

import megray_b200 as mr
from megray_b200 import _lib
from test_cpu_reduce import NP, cpu_reduce_n, make


def ring(arrays, dtype_code, op):
    lib = _lib.load()
    n = len(arrays)
    outs = [np.empty_like(arrays[0]) for _ in range(n)]
    ip = (C.c_void_p * n)(*[a.ctypes.data for a in arrays])
    opp = (C.c_void_p * n)(*[o.ctypes.data for o in outs])
    assert lib.megray_oracle_ring_all_reduce(ip, opp, n, arrays[0].size, dtype_code, op) == 0
    return outs


def tree(arrays, root, dtype_code, op):
    lib = _lib.load()
    n = len(arrays)
    out = np.empty_like(arrays[0])
    ip = (C.c_void_p * n)(*[a.ctypes.data for a in arrays])
    assert lib.megray_oracle_tree_reduce(ip, C.c_void_p(out.ctypes.data), n, root, arrays[0].size, dtype_code, op) == 0
    return out


def combine(a, b, op):
    if op == mr.SUM:
        with np.errstate(over="ignore"):
            return (a + b).astype(a.dtype)
    return np.maximum(a, b) if op == mr.MAX else np.minimum(a, b)


def numpy_ring(arrays, op):
    """Chunk c ends up on rank c-1 after being combined along the ring starting at rank c."""
    n, length = len(arrays), arrays[0].size
    counts = [length // n + (1 if c < length % n else 0) for c in range(n)]
    first = np.concatenate([[0], np.cumsum(counts)])
    out = np.empty_like(arrays[0])
    for c in range(n):
        sl = slice(first[c], first[c + 1])
        acc = arrays[c][sl]
        for step in range(1, n):
            r = (c + step) % n
            acc = combine(arrays[r][sl], acc, op)  # own value first, received value second
        out[sl] = acc
    return out


def numpy_tree(arrays, root, op):
    n = len(arrays)
    acc = [arrays[(v + root) % n].copy() for v in range(n)]
    bit = 1
    while bit < n:
        for v in range(n):
            if v & (bit - 1) or v & bit or (v | bit) >= n:
                continue
            acc[v] = combine(acc[v | bit], acc[v], op)
        bit <<= 1
    return acc[0]


@pytest.mark.parametrize("dtype_code", sorted(NP))
@pytest.mark.parametrize("op", [mr.SUM, mr.MAX, mr.MIN])
@pytest.mark.parametrize("n", [1, 2, 3, 5, 8])
def test_ring_all_reduce_schedule(dtype_code, op, n):
    arrays = [make(dtype_code, 1003, 31 * n + r) for r in range(n)]  # 1003: ragged chunks
    outs = ring(arrays, dtype_code, op)
    for o in outs[1:]:
        np.testing.assert_array_equal(o, outs[0])  # every rank ends with the same bytes
    t = NP[dtype_code]
    if t != np.float16:  # numpy's float16 add rounds once too, but through float32: same result
        np.testing.assert_array_equal(outs[0], numpy_ring(arrays, op))
    rank_order = cpu_reduce_n(arrays, dtype_code, op)
    if op != mr.SUM or not np.issubdtype(t, np.floating):
        np.testing.assert_array_equal(outs[0], rank_order)
    else:
        tol = {np.float16: 2e-2, np.float32: 1e-5, np.float64: 1e-13}[t]
        np.testing.assert_allclose(outs[0].astype(np.float64), rank_order.astype(np.float64), atol=tol * n)


@pytest.mark.parametrize("dtype_code", [mr.INT32, mr.FLOAT32, mr.FLOAT64, mr.UINT8])
@pytest.mark.parametrize("op", [mr.SUM, mr.MAX])
@pytest.mark.parametrize("n,root", [(1, 0), (2, 1), (3, 0), (5, 3), (8, 0), (8, 5)])
def test_tree_reduce_schedule(dtype_code, op, n, root):
    arrays = [make(dtype_code, 777, 17 * n + r) for r in range(n)]
    got = tree(arrays, root, dtype_code, op)
    np.testing.assert_array_equal(got, numpy_tree(arrays, root, op))
    rank_order = cpu_reduce_n(arrays, dtype_code, op)
    t = NP[dtype_code]
    if op != mr.SUM or not np.issubdtype(t, np.floating):
        np.testing.assert_array_equal(got, rank_order)
    else:
        np.testing.assert_allclose(got.astype(np.float64), rank_order.astype(np.float64),
                                   atol=(1e-5 if t == np.float32 else 1e-13) * n)


def test_bad_arguments():
    lib = _lib.load()
    a = np.zeros(4, np.float32)
    ip = (C.c_void_p * 1)(a.ctypes.data)
    assert lib.megray_oracle_ring_all_reduce(ip, ip, 0, 4, mr.FLOAT32, mr.SUM) != 0
    assert lib.megray_oracle_tree_reduce(ip, C.c_void_p(a.ctypes.data), 1, 1, 4, mr.FLOAT32, mr.SUM) != 0
