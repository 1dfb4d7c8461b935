"""The host reduction (the oracle of the device kernels) against numpy, for every numeric dtype
and op; fp16 is checked bit-for-bit through numpy's float16, bf16 through a float32 model."""
import ctypes as C

import numpy as np
import pytest

import megray_b200 as mr
from megray_b200 import _lib

NP = {mr.INT8: np.int8, mr.UINT8: np.uint8, mr.INT32: np.int32, mr.UINT32: np.uint32,
      mr.INT64: np.int64, mr.UINT64: np.uint64, mr.FLOAT16: np.float16, mr.FLOAT32: np.float32,
      mr.FLOAT64: np.float64}


def cpu_reduce_n(arrays, dtype_code, op):
    lib = _lib.load()
    out = np.empty_like(arrays[0])
    ptrs = (C.c_void_p * len(arrays))(*[a.ctypes.data for a in arrays])
    rc = lib.megray_cpu_reduce_n(ptrs, len(arrays), out.ctypes.data, arrays[0].size, dtype_code, op)
    assert rc == 0
    return out


def make(dtype_code, n, seed):
    rng = np.random.default_rng(seed)
    t = NP[dtype_code]
    if np.issubdtype(t, np.floating):
        return rng.uniform(-1, 1, n).astype(t)
    lo, hi = (-100, 100) if np.issubdtype(t, np.signedinteger) else (0, 200)
    return rng.integers(lo, hi, n).astype(t)


@pytest.mark.parametrize("dtype_code", sorted(NP))
@pytest.mark.parametrize("op", [mr.SUM, mr.MAX, mr.MIN])
@pytest.mark.parametrize("nin", [1, 2, 3, 8])
def test_matches_numpy(dtype_code, op, nin):
    arrays = [make(dtype_code, 1000 + 7, 100 * nin + r) for r in range(nin)]
    got = cpu_reduce_n(arrays, dtype_code, op)
    t = NP[dtype_code]
    if op == mr.SUM:
        if t == np.float16:  # widened to fp32, combined in order, rounded once
            acc = arrays[0].astype(np.float32)
            for a in arrays[1:]:
                acc = acc + a.astype(np.float32)
            want = acc.astype(np.float16)
        else:
            want = arrays[0].copy()
            with np.errstate(over="ignore"):
                for a in arrays[1:]:
                    want = (want + a).astype(t)
    else:
        f = np.maximum if op == mr.MAX else np.minimum
        want = arrays[0].copy()
        for a in arrays[1:]:
            want = f(want, a)
    np.testing.assert_array_equal(got, want)


def test_integer_sum_wraps():
    a = np.array([127, -128, 100], dtype=np.int8)
    b = np.array([1, -1, 100], dtype=np.int8)
    np.testing.assert_array_equal(cpu_reduce_n([a, b], mr.INT8, mr.SUM), np.array([-128, 127, -56], dtype=np.int8))


def test_bf16_sum_is_fp32_accumulate_round_once():
    rng = np.random.default_rng(0)
    f = [rng.uniform(-1, 1, 4096).astype(np.float32) for _ in range(4)]

    def to_bf16(x):  # round to nearest even
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
        return u.astype(np.uint16)

    def from_bf16(b):
        return (b.astype(np.uint32) << 16).view(np.float32)

    b = [to_bf16(x) for x in f]
    got = cpu_reduce_n(b, mr.BFLOAT16, mr.SUM)
    acc = from_bf16(b[0])
    for x in b[1:]:
        acc = acc + from_bf16(x)
    np.testing.assert_array_equal(got, to_bf16(acc))


def test_char_is_rejected_for_reductions():
    lib = _lib.load()
    a = np.zeros(4, np.uint8)
    ptrs = (C.c_void_p * 1)(a.ctypes.data)
    assert lib.megray_cpu_reduce_n(ptrs, 1, a.ctypes.data, 4, mr.CHAR, mr.SUM) == 6


def test_scale_cast_model():
    lib = _lib.load()
    xs = [np.linspace(-2, 2, 257, dtype=np.float32) * (r + 1) for r in range(3)]
    out = np.empty(257, np.float16)
    ptrs = (C.c_void_p * 3)(*[x.ctypes.data for x in xs])
    assert lib.megray_cpu_reduce_scale_cast(ptrs, 3, mr.FLOAT32, out.ctypes.data, mr.FLOAT16, 257, mr.SUM,
                                            C.c_double(1 / 3)) == 0
    want = ((xs[0] + xs[1] + xs[2]) * np.float32(1 / 3)).astype(np.float16)
    np.testing.assert_array_equal(out, want)


def test_dtype_sizes():
    lib = _lib.load()
    sizes = {mr.INT8: 1, mr.UINT8: 1, mr.INT32: 4, mr.UINT32: 4, mr.INT64: 8, mr.UINT64: 8,
             mr.FLOAT16: 2, mr.FLOAT32: 4, mr.FLOAT64: 8, mr.CHAR: 1, mr.BFLOAT16: 2}
    for code, size in sizes.items():
        assert lib.megray_dtype_size(code) == size
    assert lib.megray_dtype_size(99) == 0
