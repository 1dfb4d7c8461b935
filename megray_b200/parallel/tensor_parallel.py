"""Sequence-parallel tensor parallelism: all_gather -> GEMM and GEMM -> reduce_scatter.

Activations between the tensor-parallel regions are sharded on tokens ([T/n, d] per rank).
``TensorParallelOps`` owns the symmetric-heap buffers the two patterns need and offers them
in two forms:

* unfused: the native all_gather / reduce_scatter kernels followed / preceded by the GEMM;
* fused (``fused=True``): the gather runs as a few CTAs on a side stream and publishes one
  readiness counter per source shard; the GEMM's TMA producer waits for the counter of the
  shard that owns its rows and starts with the local shard, so transfer and math overlap
  tile by tile.  For GEMM -> reduce_scatter the GEMM epilogue stores each partial tile
  straight into the owning rank's staging slot over NVLink, and a reduce kernel sums the
  slots in rank order.

The reference library offers only the bare collectives (all_gather / reduce_scatter,
include/megray/communicator.h:79-95); composing them with matrix products is left to its user.
"""
from __future__ import annotations

import torch

from ..ops import EPI_DSWIGLU, EPI_SWIGLU, gemm


class TensorParallelOps:
    def __init__(self, comm, tokens: int, width: int, fused: bool = True):
        self.comm, self.n, self.rank = comm, comm.nranks, comm.rank
        self.T, self.d = tokens, width
        self.Ts = tokens // self.n
        self.fused = fused

    def full_buffer(self) -> torch.Tensor:
        """An all-token [T, d] bf16 buffer (gather target or partial-sum source)."""
        return torch.empty(self.T, self.d, dtype=torch.bfloat16, device="cuda")

    def _shard(self, full):
        return full[self.rank * self.Ts:(self.rank + 1) * self.Ts]

    # xg holds this rank's rows already; gather the others in place, then
    # [G|U], H = swiglu(xg @ w_gu^T)
    def ag_gemm_swiglu(self, xg, w_gu, gu, h, fl):
        self.comm.all_gather(self._shard(xg), xg)
        gemm(xg, w_gu, gu, epilogue=EPI_SWIGLU, out2=h, n=fl)

    # all_gather(dy) then dG|dU = dswiglu(dyg @ w_down)
    def ag_gemm_dswiglu(self, dy, dyg, w_down, gu, dgu, fl):
        self.comm.all_gather(dy, dyg)
        gemm(dyg, w_down, dgu, b_mn=True, epilogue=EPI_DSWIGLU, aux=gu, n=fl)

    # partial = a @ b^T (or a @ b when b_mn), then out = reduce_scatter(partial)
    def gemm_rs(self, a, b, partial, out, b_mn=False):
        gemm(a, b, partial, b_mn=b_mn)
        self.comm.reduce_scatter(partial, out)
