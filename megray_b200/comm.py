"""Python interface to the rendezvous server/client and the communicators.

Mirrors the C++ interface (``include/megray.h``): ``Server``, ``Client``,
``get_communicator(nranks, rank, backend)`` and ``Communicator.init(ip, port)``
followed by send / recv / scatter / gather / all_to_all / all_gather / all_reduce /
reduce_scatter / broadcast / reduce.  Buffers may be numpy arrays or CPU torch
tensors (host backend) or CUDA torch tensors (NCCL and NVL backends, on the
current CUDA stream unless ``stream=`` is given).  The reference library has no
Python layer; its C++ calls are ``include/megray/communicator.h:46-109``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np

from . import _lib

# enum values of include/megray/types.h
NCCL, UCX, RCCL, SHM, NVL = 0, 1, 2, 3, 4
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, CHAR, BFLOAT16 = range(11)
SUM, MAX, MIN = 0, 1, 2
OK = 0
STATUS_NAMES = [
    "OK", "SYS_ERROR", "CUDA_ERR", "NCCL_ERR", "UCX_ERR", "ENV_ERROR", "INVALID_ARGUMENT",
    "INVALID_USAGE", "UNEXPECTED_ERR", "NOT_IMPLEMENTED", "HIP_ERR", "RCCL_ERR", "TIMEOUT", "ABORTED",
    "OUT_OF_BOUNDS",
]
BACKENDS = {"nccl": NCCL, "ucx": UCX, "rccl": RCCL, "shm": SHM, "host": SHM, "nvl": NVL}
OPS = {"sum": SUM, "max": MAX, "min": MIN}

_NP_DTYPES = {
    np.dtype("int8"): INT8, np.dtype("uint8"): UINT8, np.dtype("int32"): INT32,
    np.dtype("uint32"): UINT32, np.dtype("int64"): INT64, np.dtype("uint64"): UINT64,
    np.dtype("float16"): FLOAT16, np.dtype("float32"): FLOAT32, np.dtype("float64"): FLOAT64,
}


class MegRayError(RuntimeError):
    def __init__(self, status: int, what: str):
        name = STATUS_NAMES[status] if 0 <= status < len(STATUS_NAMES) else str(status)
        super().__init__(f"{what}: {name} ({status})")
        self.status = status


def _check(status: int, what: str) -> None:
    if status != 0:
        raise MegRayError(status, what)


def _torch():
    import torch

    return torch


def _torch_dtype_code(dt) -> int:
    torch = _torch()
    table = {
        torch.int8: INT8, torch.uint8: UINT8, torch.int32: INT32, torch.int64: INT64,
        torch.float16: FLOAT16, torch.float32: FLOAT32, torch.float64: FLOAT64,
        torch.bfloat16: BFLOAT16,
    }
    for name, code in (("uint32", UINT32), ("uint64", UINT64)):
        if hasattr(torch, name):
            table[getattr(torch, name)] = code
    return table[dt]


class _Buf:
    """Pointer, element count, dtype code and context of a numpy array or torch tensor."""

    __slots__ = ("ptr", "numel", "dtype", "cuda", "keep")

    def __init__(self, x, dtype: Optional[int] = None):
        self.keep = x
        if x is None:
            self.ptr, self.numel, self.dtype, self.cuda = None, 0, dtype, None
            return
        if isinstance(x, np.ndarray):
            if not x.flags["C_CONTIGUOUS"]:
                raise ValueError("buffers must be contiguous")
            self.ptr = x.ctypes.data
            self.numel = x.size
            self.dtype = dtype if dtype is not None else _NP_DTYPES[x.dtype]
            self.cuda = False
            return
        if not x.is_contiguous():
            raise ValueError("buffers must be contiguous")
        self.ptr = x.data_ptr()
        self.numel = x.numel()
        self.dtype = dtype if dtype is not None else _torch_dtype_code(x.dtype)
        self.cuda = x.is_cuda


def _require(cond: bool, what: str) -> None:
    """Length / dtype contracts of include/megray/communicator.h, checked before the native call
    (which trusts them and would otherwise write past a tensor)."""
    if not cond:
        raise ValueError(what)


def _same_dtype(a: "_Buf", b: "_Buf", op: str) -> None:
    if a.ptr is not None and b.ptr is not None:
        _require(a.dtype == b.dtype, f"{op}: send and recv must have the same dtype")


def _ctx(bufs, stream):
    """(ctx_type, stream handle) for the buffers of one call."""
    cuda = [b.cuda for b in bufs if b.cuda is not None]
    if any(cuda):
        if not all(cuda):
            raise ValueError("mixing host and CUDA buffers in one call")
        torch = _torch()
        s = stream if stream is not None else torch.cuda.current_stream()
        return 1, C.c_void_p(s.cuda_stream)
    return 0, C.c_void_p(0)


def get_host_ip() -> Optional[str]:
    buf = C.create_string_buffer(64)
    return buf.value.decode() if _lib.load().megray_get_host_ip(buf, 64) == 0 else None


def get_free_port() -> int:
    return _lib.load().megray_get_free_port()


def create_server(nranks: int, port: int) -> None:
    """Start a detached-lifetime server (lives until rank 0 disconnects), as the reference's
    ``create_server`` does (include/megray/server.h:24)."""
    _check(_lib.load().megray_create_server(nranks, port), "create_server")


class Server:
    """Rendezvous server owned by this object (``port=0`` picks a free port)."""

    def __init__(self, nranks: int, port: int = 0):
        self._lib = _lib.load()
        self._h = self._lib.megray_server_new(nranks, port)
        if not self._h:
            raise MegRayError(1, "Server")

    @property
    def port(self) -> int:
        return self._lib.megray_server_port(self._h)

    @property
    def running(self) -> bool:
        return bool(self._lib.megray_server_running(self._h))

    @property
    def status(self) -> int:
        return self._lib.megray_server_status(self._h)

    @property
    def requests_served(self) -> int:
        return self._lib.megray_server_requests(self._h)

    def stop(self) -> None:
        self._lib.megray_server_stop(self._h)

    def close(self) -> None:
        if self._h:
            self._lib.megray_server_delete(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Client:
    """Rendezvous client (barrier / broadcast / allgather of small host blobs)."""

    def __init__(self, nranks: int, rank: int, timeout_ms: Optional[int] = None):
        self._lib = _lib.load()
        self.nranks, self.rank = nranks, rank
        self._h = self._lib.megray_client_new(nranks, rank)
        if timeout_ms is not None:
            self._lib.megray_client_set_timeout_ms(self._h, timeout_ms)

    def connect(self, ip: str, port: int) -> None:
        _check(self._lib.megray_client_connect(self._h, ip.encode(), port), "Client.connect")

    def barrier(self) -> None:
        _check(self._lib.megray_client_barrier(self._h), "Client.barrier")

    def broadcast(self, data: bytes, length: int, root: int) -> bytes:
        out = C.create_string_buffer(length)
        src = C.create_string_buffer(data, length) if self.rank == root else None
        _check(self._lib.megray_client_broadcast(self._h, src, out, length, root), "Client.broadcast")
        return out.raw

    def allgather(self, data: bytes) -> bytes:
        out = C.create_string_buffer(len(data) * self.nranks)
        _check(self._lib.megray_client_allgather(self._h, data, out, len(data)), "Client.allgather")
        return out.raw

    def close(self) -> None:
        if self._h:
            self._lib.megray_client_delete(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Communicator:
    """One rank of a communicator group.  See the module docstring for buffer rules.

    Length contracts follow ``include/megray/communicator.h``: e.g. ``all_gather`` needs
    ``recv.numel() == nranks * send.numel()``.
    """

    def __init__(self, nranks: int, rank: int, backend="nvl"):
        self._lib = _lib.load()
        self.nranks, self.rank = nranks, rank
        code = BACKENDS[backend] if isinstance(backend, str) else int(backend)
        self._h = self._lib.megray_comm_new(nranks, rank, code)
        if not self._h:
            raise MegRayError(7, "get_communicator: unknown backend")
        self.backend = code

    def init(self, ip: str, port: int) -> "Communicator":
        _check(self._lib.megray_comm_init(self._h, ip.encode(), port), "Communicator.init")
        return self

    def close(self) -> None:
        if self._h:
            self._lib.megray_comm_delete(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- state ---------------------------------------------------------------------------
    @property
    def status(self) -> int:
        return self._lib.megray_comm_status(self._h)

    def abort(self) -> None:
        self._lib.megray_comm_abort(self._h)

    def stats(self) -> dict:
        out = (C.c_uint64 * 10)()
        self._lib.megray_comm_stats(self._h, out)
        keys = ["calls", "bytes", "kernels", "timeouts", "oneshot", "twoshot", "nvls", "copy", "ll", "direct"]
        return dict(zip(keys, [int(v) for v in out]))

    # -- operations ------------------------------------------------------------------------
    def send(self, buf, peer: int, dtype=None, stream=None) -> None:
        b = _Buf(buf, dtype)
        ct, st = _ctx([b], stream)
        _check(self._lib.megray_send(self._h, b.ptr, b.numel, b.dtype, peer, ct, st), "send")

    def recv(self, buf, peer: int, dtype=None, stream=None) -> None:
        b = _Buf(buf, dtype)
        ct, st = _ctx([b], stream)
        _check(self._lib.megray_recv(self._h, b.ptr, b.numel, b.dtype, peer, ct, st), "recv")

    def scatter(self, send, recv, root: int, stream=None) -> None:
        r = _Buf(recv)
        s = _Buf(send, r.dtype)
        _same_dtype(s, r, "scatter")
        _require(r.ptr is not None, "scatter: every rank needs a recv buffer")
        if self.rank == root:
            _require(s.ptr is not None and s.numel == self.nranks * r.numel,
                     "scatter: the root's send buffer must hold nranks * recv.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_scatter(self._h, s.ptr, r.ptr, r.numel, r.dtype, root, ct, st), "scatter")

    def gather(self, send, recv, root: int, stream=None) -> None:
        s = _Buf(send)
        r = _Buf(recv, s.dtype)
        _same_dtype(s, r, "gather")
        _require(s.ptr is not None, "gather: every rank needs a send buffer")
        if self.rank == root:
            _require(r.ptr is not None and r.numel == self.nranks * s.numel,
                     "gather: the root's recv buffer must hold nranks * send.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_gather(self._h, s.ptr, r.ptr, s.numel, s.dtype, root, ct, st), "gather")

    def all_to_all(self, send, recv, stream=None) -> None:
        s, r = _Buf(send), _Buf(recv)
        _same_dtype(s, r, "all_to_all")
        _require(s.numel % self.nranks == 0 and r.numel == s.numel,
                 "all_to_all: send and recv must hold the same multiple of nranks elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_all_to_all(self._h, s.ptr, r.ptr, s.numel // self.nranks, s.dtype, ct, st),
               "all_to_all")

    def all_gather(self, send, recv, stream=None) -> None:
        s, r = _Buf(send), _Buf(recv)
        _same_dtype(s, r, "all_gather")
        _require(r.numel == self.nranks * s.numel, "all_gather: recv must hold nranks * send.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_all_gather(self._h, s.ptr, r.ptr, s.numel, s.dtype, ct, st), "all_gather")

    def all_reduce(self, send, recv, op="sum", stream=None) -> None:
        s, r = _Buf(send), _Buf(recv)
        _same_dtype(s, r, "all_reduce")
        _require(r.numel == s.numel, "all_reduce: send and recv must hold the same number of elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_all_reduce(self._h, s.ptr, r.ptr, s.numel, s.dtype, _op(op), ct, st),
               "all_reduce")

    def reduce_scatter(self, send, recv, op="sum", stream=None) -> None:
        s, r = _Buf(send), _Buf(recv)
        _same_dtype(s, r, "reduce_scatter")
        _require(s.numel == self.nranks * r.numel, "reduce_scatter: send must hold nranks * recv.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_reduce_scatter(self._h, s.ptr, r.ptr, r.numel, s.dtype, _op(op), ct, st),
               "reduce_scatter")

    def broadcast(self, send, recv, root: int, stream=None) -> None:
        r = _Buf(recv)
        s = _Buf(send, r.dtype)
        _same_dtype(s, r, "broadcast")
        _require(r.ptr is not None, "broadcast: every rank needs a recv buffer")
        if self.rank == root:
            _require(s.ptr is not None and s.numel == r.numel,
                     "broadcast: the root's send buffer must hold recv.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_broadcast(self._h, s.ptr, r.ptr, r.numel, r.dtype, root, ct, st), "broadcast")

    def reduce(self, send, recv, root: int, op="sum", stream=None) -> None:
        s = _Buf(send)
        r = _Buf(recv, s.dtype)
        _same_dtype(s, r, "reduce")
        _require(s.ptr is not None, "reduce: every rank needs a send buffer")
        if self.rank == root:
            _require(r.ptr is not None and r.numel == s.numel,
                     "reduce: the root's recv buffer must hold send.numel elements")
        ct, st = _ctx([s, r], stream)
        _check(self._lib.megray_reduce(self._h, s.ptr, r.ptr, s.numel, s.dtype, _op(op), root, ct, st),
               "reduce")

    def group_start(self) -> None:
        _check(self._lib.megray_group_start(self._h), "group_start")

    def group_end(self) -> None:
        _check(self._lib.megray_group_end(self._h), "group_end")

    # -- host backend ----------------------------------------------------------------------
    def host_barrier(self) -> None:
        _check(self._lib.megray_host_barrier(self._h), "host_barrier")

    def set_host_timeout_ms(self, ms: int) -> None:
        self._lib.megray_host_set_timeout_ms(self._h, ms)

    # -- native NVLink backend ---------------------------------------------------------------
    def sym_empty(self, shape, dtype):
        """A CUDA tensor living in this rank's symmetric heap.  Collective: every rank must call
        it with the same shape/dtype in the same order (offsets then agree on all ranks)."""
        torch = _torch()
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        numel = 1
        for s in shape:
            numel *= s
        itemsize = torch.empty(0, dtype=dtype).element_size()
        nbytes = max(numel * itemsize, 16)
        off = C.c_size_t(0)
        ptr = self._lib.megray_nvl_alloc(self._h, nbytes, C.byref(off))
        if not ptr:
            raise MegRayError(6, "sym_empty: symmetric heap exhausted or not an NVL communicator")
        t = _tensor_from_ptr(ptr, nbytes, torch.cuda.current_device()).view(dtype)[:numel].view(shape)
        t._megray_heap_offset = off.value
        return t

    def sym_free(self, tensor) -> None:
        _check(self._lib.megray_nvl_free(self._h, C.c_void_p(tensor.data_ptr())), "sym_free")

    def register(self, tensor) -> bool:
        """Collective.  Makes an ordinary CUDA tensor (not from ``sym_empty``) directly reachable
        by the peers' kernels, so that collectives on it (and on views that start at the same
        distance from its beginning on every rank) take the single-pass paths.  Every rank
        registers its own tensor of the same size, in the same order.  Returns False, on every
        rank, when some rank's memory cannot be shared (the staged paths keep working)."""
        rc = self._lib.megray_nvl_register(self._h, C.c_void_p(tensor.data_ptr()),
                                           tensor.numel() * tensor.element_size())
        if rc == 9:  # MEGRAY_NOT_IMPLEMENTED: no IPC handle for this memory
            return False
        _check(rc, "register")
        return True

    def deregister(self, tensor) -> None:
        """Collective.  Drops the registration made with :meth:`register`."""
        _check(self._lib.megray_nvl_deregister(self._h, C.c_void_p(tensor.data_ptr())), "deregister")

    def peer_ptr(self, tensor, peer: int) -> int:
        p = self._lib.megray_nvl_peer_ptr(self._h, C.c_void_p(tensor.data_ptr()), peer)
        if not p:
            raise MegRayError(6, "peer_ptr: tensor is not in the symmetric heap")
        return p

    def heap_base(self, peer: int) -> int:
        return self._lib.megray_nvl_heap_base(self._h, peer) or 0

    def all_reduce_scaled(self, send, recv, scale: float, op="sum", stream=None) -> None:
        """recv = cast(scale * reduce(send)): input and output dtypes may differ (bf16/fp16/fp32)."""
        s, r = _Buf(send), _Buf(recv)
        _require(r.numel == s.numel, "all_reduce_scaled: send and recv must hold the same number of elements")
        _, st = _ctx([s, r], stream)
        _check(self._lib.megray_nvl_all_reduce_scaled(self._h, s.ptr, r.ptr, s.numel, s.dtype, r.dtype,
                                                      C.c_float(scale), _op(op), st), "all_reduce_scaled")

    def stream_barrier(self, stream=None) -> None:
        torch = _torch()
        s = stream if stream is not None else torch.cuda.current_stream()
        _check(self._lib.megray_nvl_stream_barrier(self._h, C.c_void_p(s.cuda_stream)), "stream_barrier")

    def set_device_timeout_ms(self, ms: int) -> None:
        self._lib.megray_nvl_set_device_timeout_ms(self._h, ms)

    def check_canaries(self) -> None:
        """Synchronises the device and verifies the guard zones around the staging workspaces;
        raises MegRayError(OUT_OF_BOUNDS) if a kernel wrote into one."""
        _check(self._lib.megray_nvl_check_canaries(self._h), "check_canaries")

    def set_p2p_async(self, on: bool = True) -> None:
        """send / recv run on a stream of the communicator's own.  By default the caller's stream
        waits for each transfer (stream-ordered, as the interface says); with ``on`` that wait is
        postponed to :meth:`p2p_join`, so that kernels enqueued in between overlap the transfer."""
        self._lib.megray_nvl_set_p2p_async(self._h, 1 if on else 0)

    def p2p_join(self, stream=None) -> None:
        torch = _torch()
        s = stream if stream is not None else torch.cuda.current_stream()
        _check(self._lib.megray_nvl_p2p_join(self._h, C.c_void_p(s.cuda_stream)), "p2p_join")


def _op(op) -> int:
    return OPS[op] if isinstance(op, str) else int(op)


class _RawCuda:
    """Exposes raw device memory through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2, "strides": None,
        }


def _tensor_from_ptr(ptr: int, nbytes: int, device: int):
    torch = _torch()
    return torch.as_tensor(_RawCuda(ptr, nbytes), device=torch.device("cuda", device))


def get_communicator(nranks: int, rank: int, backend="nvl") -> Communicator:
    return Communicator(nranks, rank, backend)
