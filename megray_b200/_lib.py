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
        ("variant", C.c_int),
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


def _declare(lib) -> None:
    """argtypes / restype of the C interface (include/megray/c_api.h)."""
    vp, u32, u64, i32, i64, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int, C.c_int64, C.c_size_t
    P = C.POINTER

    def d(name, res, *args):
        f = getattr(lib, name)
        f.restype = res
        f.argtypes = list(args)

    d("megray_get_host_ip", i32, C.c_char_p, sz)
    d("megray_get_free_port", i32)
    d("megray_create_server", i32, u32, i32)
    d("megray_server_new", vp, u32, i32)
    d("megray_server_port", i32, vp)
    d("megray_server_running", i32, vp)
    d("megray_server_status", i32, vp)
    d("megray_server_requests", u64, vp)
    d("megray_server_stop", None, vp)
    d("megray_server_delete", None, vp)
    d("megray_client_new", vp, u32, u32)
    d("megray_client_set_timeout_ms", None, vp, i64)
    d("megray_client_connect", i32, vp, C.c_char_p, i32)
    d("megray_client_barrier", i32, vp)
    d("megray_client_broadcast", i32, vp, vp, vp, sz, u32)
    d("megray_client_allgather", i32, vp, vp, vp, sz)
    d("megray_client_delete", None, vp)
    d("megray_comm_new", vp, u32, u32, i32)
    d("megray_comm_delete", None, vp)
    d("megray_comm_init", i32, vp, C.c_char_p, i32)
    d("megray_comm_backend", i32, vp)
    d("megray_comm_status", i32, vp)
    d("megray_comm_abort", None, vp)
    d("megray_comm_stats", None, vp, P(u64))
    d("megray_send", i32, vp, vp, sz, i32, u32, i32, vp)
    d("megray_recv", i32, vp, vp, sz, i32, u32, i32, vp)
    d("megray_scatter", i32, vp, vp, vp, sz, i32, u32, i32, vp)
    d("megray_gather", i32, vp, vp, vp, sz, i32, u32, i32, vp)
    d("megray_all_to_all", i32, vp, vp, vp, sz, i32, i32, vp)
    d("megray_all_gather", i32, vp, vp, vp, sz, i32, i32, vp)
    d("megray_all_reduce", i32, vp, vp, vp, sz, i32, i32, i32, vp)
    d("megray_reduce_scatter", i32, vp, vp, vp, sz, i32, i32, i32, vp)
    d("megray_broadcast", i32, vp, vp, vp, sz, i32, u32, i32, vp)
    d("megray_reduce", i32, vp, vp, vp, sz, i32, i32, u32, i32, vp)
    d("megray_group_start", i32, vp)
    d("megray_group_end", i32, vp)
    d("megray_host_barrier", i32, vp)
    d("megray_host_set_timeout_ms", None, vp, i64)
    d("megray_nvl_alloc", vp, vp, sz, P(sz))
    d("megray_nvl_free", i32, vp, vp)
    d("megray_nvl_peer_ptr", vp, vp, vp, u32)
    d("megray_nvl_register", i32, vp, vp, C.c_size_t)
    d("megray_nvl_deregister", i32, vp, vp)
    d("megray_nvl_heap_base", vp, vp, u32)
    d("megray_nvl_heap_bytes", sz, vp)
    d("megray_nvl_all_reduce_scaled", i32, vp, vp, vp, sz, i32, i32, C.c_float, i32, vp)
    d("megray_nvl_stream_barrier", i32, vp, vp)
    d("megray_nvl_set_device_timeout_ms", None, vp, i64)
    d("megray_nvl_check_canaries", i32, vp)
    d("megray_nvl_set_p2p_async", None, vp, i32)
    d("megray_nvl_p2p_join", i32, vp, vp)
    d("megray_cpu_reduce_n", i32, P(vp), i32, vp, sz, i32, i32)
    d("megray_cpu_reduce_scale_cast", i32, P(vp), i32, i32, vp, i32, sz, i32, C.c_double)
    d("megray_oracle_ring_all_reduce", i32, P(vp), P(vp), i32, sz, i32, i32)
    d("megray_oracle_tree_reduce", i32, P(vp), vp, i32, i32, sz, i32, i32)
    d("megray_gemm_tile_schedule", i32, C.POINTER(GemmArgs), i32, P(i32), i32)
    d("megray_reduce_n", i32, P(vp), i32, vp, sz, i32, i32, i32, C.c_float, vp)
    d("megray_sgd_bf16", i32, vp, vp, vp, u64, C.c_float, C.c_float, C.c_float, vp)
    d("megray_mse_bf16", i32, vp, vp, vp, vp, u64, C.c_float, vp)
    d("megray_add_rmsnorm_bf16", i32, vp, vp, vp, vp, vp, i32, i32, C.c_float, vp)
    d("megray_rmsnorm_bwd_bf16", i32, vp, vp, vp, vp, vp, i32, i32, vp)
    d("megray_tp_ag_gemm", i32, vp, P(GemmArgs), vp, vp, vp, vp)
    d("megray_tp_gemm_rs", i32, vp, P(GemmArgs), vp, vp, vp, vp, C.c_size_t, vp)
    d("megray_tp_rs_counter_bytes", C.c_size_t, i32, i32)
    d("megray_moe_route", i32, vp, i32, i32, vp, vp, vp, vp)
    d("megray_moe_route_bwd", i32, vp, vp, vp, i32, i32, vp, vp)
    d("megray_moe_plan", i32, vp, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp, vp)
    d("megray_moe_plan_exchange", i32, vp, vp, i32, i32, vp, vp, vp, vp, vp, vp, vp)
    d("megray_moe_zero_pads", i32, vp, i32, vp, vp, vp, i32, vp)
    d("megray_moe_dispatch", i32, vp, i32, i32, vp, vp, vp, vp, vp, vp, P(vp), i32, i32, i32, vp)
    d("megray_moe_combine", i32, vp, i32, i32, vp, vp, vp, P(vp), i32, i32, i32, vp)
    d("megray_moe_combine_dw", i32, vp, i32, i32, vp, vp, P(vp), i32, i32, i32, vp, vp)
    d("megray_dtype_size", sz, i32)
    d("megray_set_log_level", None, i32)
    d("megray_trace_enable", None, C.c_char_p)
    d("megray_trace_dump", sz)


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
        _declare(lib)
        _lib = lib
        return lib
