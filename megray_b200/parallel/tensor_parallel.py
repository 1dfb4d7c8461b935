"""Sequence-parallel tensor parallelism: all_gather -> GEMM and GEMM -> reduce_scatter.

Activations between the tensor-parallel regions are sharded on tokens ([T/n, d] per rank).
``TensorParallelOps`` owns the symmetric-heap buffers the two patterns need and offers them
in two forms:

* unfused: the native all_gather / reduce_scatter kernels followed / preceded by the GEMM;
* fused (``fused=True``): the gather runs as a few CTAs on a side stream and publishes one
  readiness counter per source shard; the GEMM's TMA producer waits for the counter of the
  shard that owns its rows and starts with the local shard, so transfer and math overlap
  tile by tile.  For GEMM -> reduce_scatter the GEMM epilogue stores each partial tile of
  another rank's rows straight into that rank's staging slot over NVLink; the tiles of the
  rank's own rows come last and add the staged partials in their epilogue (rank order).

The reference library offers only the bare collectives (all_gather / reduce_scatter,
include/megray/communicator.h:79-95); composing them with matrix products is left to its user.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib
from ..ops import EPI_DSWIGLU, EPI_SWIGLU, build_gemm_args, gemm


class TensorParallelOps:
    """Owns the symmetric-heap buffers of one tensor-parallel region over [tokens, width]
    activations.  Every rank must create it, and ask it for buffers, in the same order."""

    def __init__(self, comm, tokens: int, width: int, fused: bool = True):
        self.comm, self.n, self.rank = comm, comm.nranks, comm.rank
        self.T, self.d = tokens, width
        self.Ts = tokens // self.n
        self.fused = fused and self.Ts % 256 == 0
        # SMs the GEMMs may occupy (0 = all); lower it to leave room for kernels of other streams
        self.sm_limit = 0
        # GEMM tile variant (0 = chosen by the library; 2 = 256-row CTA-pair tile, 3 = 512-row tile)
        self.variant = 0
        self._lib = _lib.load()
        self._stage = []
        self._parity = 0
        if self.fused:
            # partial-sum staging: n slots of [T/n, d], double-buffered by call parity
            words = self._lib.megray_tp_rs_counter_bytes(self.Ts, width) // 4
            for _ in range(2):
                st = comm.sym_empty((tokens, width), torch.bfloat16)
                # one delivery counter per 32 rows x 256 columns of this rank's shard
                st._tp_counters = comm.sym_empty((words,), torch.int32)
                st._tp_counters.zero_()
                self._stage.append(st)
            self._settle()

    # -- buffers -----------------------------------------------------------------------------
    def _flag_block(self) -> torch.Tensor:
        f = self.comm.sym_empty((64,), torch.int32)  # 256 bytes
        f.zero_()
        return f

    def _settle(self) -> None:
        """Flag blocks are zeroed on every rank before any rank's kernel may write into them."""
        torch.cuda.synchronize()
        self.comm.stream_barrier()
        torch.cuda.synchronize()

    def full_buffer(self) -> torch.Tensor:
        """An all-token [T, d] bf16 buffer in the symmetric heap (gather target)."""
        if not self.fused:
            return torch.empty(self.T, self.d, dtype=torch.bfloat16, device="cuda")
        t = self.comm.sym_empty((self.T, self.d), torch.bfloat16)
        t._tp_flags = self._flag_block()
        self._settle()
        return t

    def shard_buffer(self) -> torch.Tensor:
        """A [T/n, d] bf16 buffer peers can read (source of a fused gather)."""
        if not self.fused:
            return torch.empty(self.Ts, self.d, dtype=torch.bfloat16, device="cuda")
        return self.comm.sym_empty((self.Ts, self.d), torch.bfloat16)

    def _shard(self, full):
        return full[self.rank * self.Ts:(self.rank + 1) * self.Ts]

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    # -- all_gather -> GEMM ------------------------------------------------------------------
    def _ag_gemm(self, src, full, args):
        rc = self._lib.megray_tp_ag_gemm(self.comm._h, C.byref(args), full.data_ptr(), src.data_ptr(),
                                         full._tp_flags.data_ptr(), self._stream())
        if rc != 0:
            raise RuntimeError(f"megray_tp_ag_gemm failed ({rc})")

    def ag_gemm_swiglu(self, xg, w_gu, gu, h, fl):
        """xg holds this rank's rows already; gather the others (in place) while computing
        [G|U], H = swiglu(xg @ w_gu^T)."""
        if not self.fused:
            self.comm.all_gather(self._shard(xg), xg)
            gemm(xg, w_gu, gu, epilogue=EPI_SWIGLU, out2=h, n=fl, sm_limit=self.sm_limit)
            return
        args, _, _ = build_gemm_args(xg, w_gu, gu, epilogue=EPI_SWIGLU, out2=h, n=fl, sm_limit=self.sm_limit,
                                     variant=self.variant)
        self._ag_gemm(self._shard(xg), xg, args)

    def ag_gemm_dswiglu(self, dy, dyg, w_down, gu, dgu, fl):
        """dyg = all_gather(dy) while computing dG|dU = dswiglu(dyg @ w_down)."""
        if not self.fused:
            self.comm.all_gather(dy, dyg)
            gemm(dyg, w_down, dgu, b_mn=True, epilogue=EPI_DSWIGLU, aux=gu, n=fl, sm_limit=self.sm_limit)
            return
        args, _, _ = build_gemm_args(dyg, w_down, dgu, b_mn=True, epilogue=EPI_DSWIGLU, aux=gu, n=fl,
                                     sm_limit=self.sm_limit, variant=self.variant)
        self._ag_gemm(dy, dyg, args)

    # -- GEMM -> reduce_scatter --------------------------------------------------------------
    def gemm_rs(self, a, b, partial, out, b_mn=False, residual=None):
        """out[T/n, d] = reduce_scatter(a @ b^T) (a @ b when b_mn) (+ residual)."""
        if not self.fused:
            gemm(a, b, partial, b_mn=b_mn, sm_limit=self.sm_limit)
            self.comm.reduce_scatter(partial, out)
            if residual is not None:
                out.add_(residual)
            return
        st = self._stage[self._parity]
        self._parity ^= 1
        args, _, _ = build_gemm_args(a, b, None, b_mn=b_mn, alloc_out=False, sm_limit=self.sm_limit,
                                     variant=self.variant)
        rc = self._lib.megray_tp_gemm_rs(self.comm._h, C.byref(args), st.data_ptr(), out.data_ptr(),
                                         residual.data_ptr() if residual is not None else None,
                                         st._tp_counters.data_ptr(), st._tp_counters.numel() * 4, self._stream())
        if rc != 0:
            raise RuntimeError(f"megray_tp_gemm_rs failed ({rc})")
