"""ctypes loader for ``libmegray.so`` and the C structures of its interface."""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libmegray.so")

_lib = None
_lock = threading.Lock()


class GemmArgs(C.Structure):
    """Mirror of ``megray_gemm_args`` (include/megray/c_api.h)."""

    _fields_ = [
        ("A", C.c_void_p),
        ("B", C.c_void_p),
        ("D", C.c_void_p),
        ("D2", C.c_void_p),
        ("aux", C.c_void_p),
        ("M", C.c_int),
        ("N", C.c_int),
        ("K", C.c_int),
        ("lda", C.c_int64),
        ("ldb", C.c_int64),
        ("ldd", C.c_int64),
        ("ldd2", C.c_int64),
        ("ldaux", C.c_int64),
        ("a_mn", C.c_int),
        ("b_mn", C.c_int),
        ("epilogue", C.c_int),
        ("aux_off", C.c_int),
        ("m_rot", C.c_int),
        ("sm_limit", C.c_int),
        ("a_ready", C.c_void_p),
        ("rows_per_flag", C.c_int),
        ("a_ready_target", C.c_uint32),
        ("peer_out", C.c_void_p),
        ("rows_per_peer", C.c_int),
        ("m_block_group", C.c_void_p),
        ("group_rows_b", C.c_int),
        ("k_begin", C.c_void_p),
        ("k_end", C.c_void_p),
        ("groups", C.c_int),
        ("error_flag", C.c_void_p),
        ("wait_limit_ns", C.c_uint64),
    ]


def load(build_if_missing: bool = True) -> C.CDLL:
    """Load the native library (building it first when it is absent)."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            if not build_if_missing:
                raise OSError(f"{LIB_PATH} is missing: run `python -m megray_b200.build`")
            from . import build as _build

            _build.build()
        lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        lib.megray_gemm_bf16.argtypes = [C.POINTER(GemmArgs), C.c_void_p]
        lib.megray_gemm_bf16.restype = C.c_int
        lib.megray_launch_count.argtypes = []
        lib.megray_launch_count.restype = C.c_uint64
        _lib = lib
        return lib
