"""bf16 GEMM on the library's tcgen05 kernel (src/kernels/gemm_tcgen05.cu).

``gemm(a, b)`` computes ``D[M, N] = A[M, K] @ B[N, K]^T`` with fp32 accumulation.  Each
operand can instead be given in its transposed storage ("MN-major"): ``a_mn=True`` means
``a`` is stored ``[K, M]``, ``b_mn=True`` means ``b`` is stored ``[K, N]``; the kernel reads
either through TMA without any transposition pass.  Epilogues:

* ``EPI_STORE``   D = acc
* ``EPI_ACCUM``   D += acc
* ``EPI_STORE_ROWS`` D = acc, written as whole 128-byte row segments staged through shared memory
* ``EPI_SWIGLU``  ``b`` = [W_gate; W_up] stacked ([2F, K]); writes G|U into ``out`` ([M, 2F]) and
                  silu(G) * U into ``out2`` ([M, F])
* ``EPI_DSWIGLU`` acc = dH ([M, F]); reads saved G|U from ``aux`` and writes dG|dU into ``out``
* ``EPI_STORE_F32`` D = acc as float32 (``out`` is a float32 tensor): partial products of a K split

There is no GEMM in the reference library; this one exists for the tensor-parallel MLP and
MoE entry points.  A missing native library or a launch failure raises: nothing here falls
back to another implementation.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

EPI_STORE, EPI_SWIGLU, EPI_DSWIGLU, EPI_ACCUM, EPI_PUSH, EPI_STORE_ROWS, EPI_STORE_F32 = 0, 1, 2, 3, 4, 5, 6

_err_flags = {}


def gemm_error_flag(device=None) -> torch.Tensor:
    """Per-device int32 word the kernels set when one of their bounded waits ran out."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = dev.index
    if key not in _err_flags:
        _err_flags[key] = torch.zeros(1, dtype=torch.int32, device=dev)
    return _err_flags[key]


def _check2d(t: torch.Tensor, name: str, dtype=torch.bfloat16) -> None:
    if t.dtype != dtype or t.dim() != 2 or not t.is_cuda:
        raise ValueError(f"{name}: expected a 2-D CUDA {dtype} tensor")
    if t.stride(1) != 1 or t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"{name}: rows must be contiguous, 16-byte aligned, leading dimension % 8 == 0")


def build_gemm_args(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, *, a_mn: bool = False,
                    b_mn: bool = False, epilogue: int = EPI_STORE, out2: torch.Tensor = None,
                    aux: torch.Tensor = None, n: int = None, sm_limit: int = 0, m_rot: int = 0,
                    a_ready: torch.Tensor = None, rows_per_flag: int = 0, a_ready_target: int = 0,
                    m_block_group: torch.Tensor = None, group_rows_b: int = 0, k_begin: torch.Tensor = None,
                    k_end: torch.Tensor = None, groups: int = 0, peer_out: torch.Tensor = None,
                    rows_per_peer: int = 0, wait_limit_ms: int = 0, variant: int = 0, alloc_out: bool = True):
    """Validates the operands and fills the C argument block; returns (args, out, out2).  The
    tensors referenced by ``args`` must stay alive until the launch has been enqueued."""
    _check2d(a, "a")
    _check2d(b, "b")
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    Nb, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    grouped = m_block_group is not None or k_begin is not None
    if not grouped and Kb != K:
        raise ValueError(f"inner dimensions differ: {K} vs {Kb}")
    if epilogue == EPI_SWIGLU:
        N = Nb // 2 if n is None else n
        aux_off = N
    else:
        N = Nb if n is None else n
        aux_off = N if epilogue == EPI_DSWIGLU else 0
    out_cols = 2 * N if epilogue in (EPI_SWIGLU, EPI_DSWIGLU) else N
    out_rows = M * groups if k_begin is not None else M
    out_dtype = torch.float32 if epilogue == EPI_STORE_F32 else torch.bfloat16
    if out is None and alloc_out:
        out = torch.empty(out_rows, out_cols, dtype=out_dtype, device=a.device)
    args = _lib.GemmArgs()
    args.A, args.B = a.data_ptr(), b.data_ptr()
    if out is not None:
        _check2d(out, "out", out_dtype)
        args.D, args.ldd = out.data_ptr(), out.stride(0)
    else:
        args.ldd = out_cols
    args.M, args.N, args.K = M, N, K
    args.lda, args.ldb = a.stride(0), b.stride(0)
    args.a_mn, args.b_mn, args.epilogue, args.aux_off = int(a_mn), int(b_mn), epilogue, aux_off
    args.m_rot, args.sm_limit, args.variant = m_rot, sm_limit, variant
    if epilogue == EPI_SWIGLU:
        if out2 is None:
            out2 = torch.empty(M, N, dtype=torch.bfloat16, device=a.device)
        _check2d(out2, "out2")
        args.D2, args.ldd2 = out2.data_ptr(), out2.stride(0)
    if epilogue == EPI_DSWIGLU:
        if aux is None:
            raise ValueError("EPI_DSWIGLU needs aux = saved [G | U]")
        _check2d(aux, "aux")
        args.aux, args.ldaux = aux.data_ptr(), aux.stride(0)
    if a_ready is not None:
        args.a_ready, args.rows_per_flag, args.a_ready_target = a_ready.data_ptr(), rows_per_flag, a_ready_target
    if m_block_group is not None:
        args.m_block_group, args.group_rows_b, args.groups = m_block_group.data_ptr(), group_rows_b, groups
    if k_begin is not None:
        args.k_begin, args.k_end, args.groups = k_begin.data_ptr(), k_end.data_ptr(), groups
    if peer_out is not None:
        args.peer_out, args.rows_per_peer = peer_out.data_ptr(), rows_per_peer
    args.error_flag = gemm_error_flag(a.device).data_ptr()
    args.wait_limit_ns = wait_limit_ms * 1_000_000
    return args, out, out2


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor = None, **kw) -> torch.Tensor:
    """See the module docstring.  Keyword arguments as for :func:`build_gemm_args`; ``n`` overrides
    the output width (needed for SWIGLU, where the logical N is F while ``b`` has 2F rows, and
    for grouped problems)."""
    args, out, out2 = build_gemm_args(a, b, out, **kw)
    rc = _lib.load().megray_gemm_bf16(C.byref(args), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"megray_gemm_bf16 failed (code {rc}) for M={args.M} N={args.N} K={args.K}")
    return (out, out2) if args.epilogue == EPI_SWIGLU else out


# ---------------------------------------------------------------------------------- split K
# A GEMM with few output tiles and a long K loop (the weight gradients of a sharded layer:
# M x N small, K = all tokens) wastes a large part of its last wave: 224 tiles on 74 CTA pairs take
# the time of 4 waves for the work of 3.03.  Cutting K into S ranges makes S times as many tiles
# of 1/S the length, which fill the waves better; each range writes its own partial result (the
# kernel's grouped-K form) and the N-way reduce kernel sums them.

_split_ranges = {}


def pick_split_k(M: int, N: int, K: int, sms: int = 148) -> int:
    """Number of K ranges (1..8) that minimises the estimated time: waves of 512 x 256 tiles on
    ``sms // 2`` CTA pairs, plus the bandwidth cost of writing and summing the partial results."""
    if M % 256 or K < 4096:
        return 1
    pairs = max(1, sms // 2)
    tile_m = 512 if M % 512 == 0 else 256
    tiles = -(-M // tile_m) * -(-N // 256)
    tile_s = 2.0 * tile_m * 256 * K / (17.5e12 if tile_m == 512 else 16e12)  # seconds, one full-K tile
    best, best_t = 1, None
    for s in range(1, 9):
        if K // s < 2048:
            break
        t = -(-tiles * s // pairs) * tile_s / s
        if s > 1:
            t += (4 * s + 1) * M * N * 2 / 5.0e12  # float32 partials written and read back, result written
        if best_t is None or t < best_t * 0.97:  # a split must pay for itself
            best, best_t = s, t
    return best


def gemm_split_k(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, splits: int, partial: torch.Tensor = None,
                 *, a_mn: bool = False, b_mn: bool = False) -> torch.Tensor:
    """``out = A @ B^T`` computed as ``splits`` partial products over disjoint K ranges (multiples
    of 64), kept in float32 and summed in float32: the result is rounded to bf16 once, like that of
    an unsplit product.  ``out`` must be contiguous; ``partial`` is an optional ``[splits * M, N]``
    float32 workspace."""
    if splits <= 1:
        return gemm(a, b, out, a_mn=a_mn, b_mn=b_mn)
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N = b.shape[1] if b_mn else b.shape[0]
    if splits > 8 or M % 256 or not out.is_contiguous() or out.shape != (M, N):
        raise ValueError("gemm_split_k: at most 8 ranges, M a multiple of 256, contiguous [M, N] output")
    per = -(-(-(-K // 64)) // splits) * 64  # ceil(ceil(K / 64) / splits) * 64
    key = (a.device.index, K, splits)
    if key not in _split_ranges:
        begin = [min(K, i * per) for i in range(splits)]
        end = [min(K, (i + 1) * per) for i in range(splits)]
        if any(e <= s for s, e in zip(begin, end)):
            raise ValueError("gemm_split_k: K is too short for this many ranges")
        _split_ranges[key] = (torch.tensor(begin, dtype=torch.int32, device=a.device),
                              torch.tensor(end, dtype=torch.int32, device=a.device))
    k_begin, k_end = _split_ranges[key]
    if partial is None:
        partial = torch.empty(splits * M, N, dtype=torch.float32, device=a.device)
    part = partial[: splits * M]
    if part.shape[1] != N or not part.is_contiguous():
        raise ValueError("gemm_split_k: the workspace must be a contiguous [>= splits * M, N] tensor")
    gemm(a, b, part, a_mn=a_mn, b_mn=b_mn, n=N, k_begin=k_begin, k_end=k_end, groups=splits,
         variant=3 if M % 512 == 0 else 2, epilogue=EPI_STORE_F32)
    ptrs = (C.c_void_p * splits)(*[part.data_ptr() + i * M * N * 4 for i in range(splits)])
    rc = _lib.load().megray_reduce_n(ptrs, splits, C.c_void_p(out.data_ptr()), M * N, 7, 10,  # float32 -> bfloat16
                                     0, C.c_float(1.0), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    if rc != 0:
        raise RuntimeError(f"megray_reduce_n failed ({rc})")
    return out
