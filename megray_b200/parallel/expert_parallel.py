"""Expert parallelism: top-2 routing, dispatch and combine fused with their all-to-all.

``ExpertParallelOps`` owns the routing state of one MoE layer on one rank:

    route(logits)            top-2 experts and gate weights per token, per-expert counts
    plan()                   one launch: exchange the counts (flagged words through the peers' small-message
                             slots) and compute where every rank's tokens land in each owner's
                             expert-sorted buffer (segments padded to 128 rows), all on the device:
                             no host synchronisation, no separate all_gather
    dispatch(src, dst, w)    every (token, slot) row is stored straight at its final position in the
                             owning GPU's buffer over NVLink: permute + all-to-all-v in one kernel
    combine(out, src, w)     every token loads its two expert rows from the GPUs that hold them and
                             forms the gate-weighted sum: all-to-all-v + un-permute + weighting in one
    combine_dw(dout, src)    gate gradients (a dot product per (token, slot))

Buffers that peers write into or read from live in the symmetric heap.  The reference's
all_to_all moves equal-sized chunks only (include/megray/communicator.h:75-77); variable counts
and the fusion with the permutation have no counterpart there.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


class ExpertParallelOps:
    def __init__(self, comm, tokens: int, hidden: int, experts: int, capacity_factor: float = 1.25):
        self.comm = comm
        self.n = comm.nranks if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        if experts % self.n:
            raise ValueError("experts must be divisible by the number of ranks")
        self.T, self.H, self.E = tokens, hidden, experts
        self.El = experts // self.n
        rows = int(tokens * 2 * capacity_factor) + self.El * 128
        self.capacity = (rows + 127) // 128 * 128
        self._lib = _lib.load()
        dev = torch.device("cuda", torch.cuda.current_device())
        i32 = dict(dtype=torch.int32, device=dev)
        self.idx = torch.empty(tokens, 2, **i32)
        self.w = torch.empty(tokens, 2, dtype=torch.float32, device=dev)
        self.pos = torch.empty(tokens, 2, **i32)
        self.counts = torch.zeros(experts, **i32)
        self.counts_all = torch.zeros(self.n, experts, **i32)
        self.cursor = torch.zeros(experts, **i32)
        self.send_base = torch.empty(experts, **i32)
        self.seg_begin = torch.empty(self.El, **i32)
        self.seg_end = torch.empty(self.El, **i32)
        self.seg_rows = torch.empty(self.El, **i32)
        self.block_group = torch.empty(self.capacity // 128, **i32)
        self.total = torch.zeros(2, **i32)

    # -- buffers -----------------------------------------------------------------------------
    def exchange_buffer(self) -> torch.Tensor:
        """A [capacity, hidden] bf16 buffer peers can write to / read from."""
        if self.comm is None:
            t = torch.zeros(self.capacity, self.H, dtype=torch.bfloat16, device="cuda")
        else:
            t = self.comm.sym_empty((self.capacity, self.H), torch.bfloat16)
            t.zero_()
        t._peers = self._peer_array(t)
        return t

    def _peer_array(self, t):
        arr = (C.c_void_p * self.n)()
        for q in range(self.n):
            arr[q] = t.data_ptr() if self.comm is None else self.comm.peer_ptr(t, q)
        return arr

    def _stream(self):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _check(self, rc, what):
        if rc != 0:
            raise RuntimeError(f"{what} failed ({rc})")

    def barrier(self) -> None:
        """Later work of every rank starts after earlier work of all ranks (stream-ordered)."""
        if self.comm is not None:
            self.comm.stream_barrier()

    # -- routing -----------------------------------------------------------------------------
    def route(self, logits: torch.Tensor) -> None:
        assert logits.dtype == torch.float32 and logits.shape == (self.T, self.E) and logits.is_contiguous()
        self.counts.zero_()
        self._check(self._lib.megray_moe_route(logits.data_ptr(), self.T, self.E, self.idx.data_ptr(),
                                               self.w.data_ptr(), self.counts.data_ptr(), self._stream()), "moe_route")

    def plan(self) -> None:
        if self.comm is not None and self.comm.backend == 4:  # NVL: counts travel inside the plan launch
            # (every rank hears from every other one here, which also orders this step after
            # every rank's previous step: the exchange buffers are re-used)
            self._check(self._lib.megray_moe_plan_exchange(
                self.comm._h, self.counts.data_ptr(), self.E, self.capacity, self.send_base.data_ptr(),
                self.seg_begin.data_ptr(), self.seg_end.data_ptr(), self.seg_rows.data_ptr(),
                self.block_group.data_ptr(), self.total.data_ptr(), self._stream()), "moe_plan_exchange")
            return
        if self.comm is not None:
            # also orders this step after every rank's previous step (buffers are re-used)
            self.comm.all_gather(self.counts, self.counts_all.view(-1))
            counts_all = self.counts_all
        else:
            counts_all = self.counts
        self._check(self._lib.megray_moe_plan(counts_all.data_ptr(), self.n, self.rank, self.E, self.capacity,
                                              self.send_base.data_ptr(), self.seg_begin.data_ptr(),
                                              self.seg_end.data_ptr(), self.seg_rows.data_ptr(),
                                              self.block_group.data_ptr(), self.total.data_ptr(), self._stream()),
                    "moe_plan")

    def route_bwd(self, dw: torch.Tensor, dlogits: torch.Tensor) -> None:
        self._check(self._lib.megray_moe_route_bwd(self.idx.data_ptr(), self.w.data_ptr(), dw.data_ptr(), self.T,
                                                   self.E, dlogits.data_ptr(), self._stream()), "moe_route_bwd")

    # -- dispatch / combine ------------------------------------------------------------------
    def zero_pads(self, buf: torch.Tensor) -> None:
        self._check(self._lib.megray_moe_zero_pads(buf.data_ptr(), self.H, self.seg_begin.data_ptr(),
                                                   self.seg_rows.data_ptr(), self.seg_end.data_ptr(), self.El,
                                                   self._stream()), "moe_zero_pads")

    def dispatch(self, src: torch.Tensor, dst: torch.Tensor, weights: bool = False, first: bool = True) -> None:
        """Rows of ``src`` [T, H] go to their experts' owners' ``dst`` buffers.  ``first=True`` assigns
        the destination rows (and remembers them); ``first=False`` re-uses them (backward).  With
        ``weights`` each row is scaled by its gate weight on the way."""
        if first:
            self.cursor.zero_()
        self._check(self._lib.megray_moe_dispatch(
            src.data_ptr(), self.T, self.H, self.idx.data_ptr(), self.w.data_ptr() if weights else None,
            self.send_base.data_ptr(), self.cursor.data_ptr(), None if first else self.pos.data_ptr(),
            self.pos.data_ptr(), dst._peers, self.n, self.El, self.capacity, self._stream()), "moe_dispatch")

    def combine(self, out: torch.Tensor, src: torch.Tensor, weights: bool = True) -> None:
        self._check(self._lib.megray_moe_combine(out.data_ptr(), self.T, self.H, self.idx.data_ptr(),
                                                 self.w.data_ptr() if weights else None, self.pos.data_ptr(),
                                                 src._peers, self.n, self.El, self.capacity, self._stream()), "moe_combine")

    def combine_dw(self, dout: torch.Tensor, src: torch.Tensor, dw: torch.Tensor) -> None:
        self._check(self._lib.megray_moe_combine_dw(dout.data_ptr(), self.T, self.H, self.idx.data_ptr(),
                                                    self.pos.data_ptr(), src._peers, self.n, self.El,
                                                    self.capacity, dw.data_ptr(), self._stream()), "moe_combine_dw")

    def overflowed(self) -> bool:
        """True if some owner's buffer was too small for its tokens (host read)."""
        return bool(self.total[1].item())
