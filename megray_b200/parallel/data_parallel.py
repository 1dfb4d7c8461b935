"""Data parallelism: bucketed gradient all_reduce fused with scale/cast, overlapped with backward.

``GradBucketer`` flattens a model's parameters and gradients into buckets (25 MB by default,
filled in reverse registration order, i.e. roughly the order gradients become ready).  Every
parameter's ``.grad`` is a view into its bucket; a post-accumulate-grad hook counts the ready
parameters of a bucket and, when the bucket is complete, launches one fused kernel on a
communication stream: ``out = (1/world) * sum over ranks`` (in place), while backward continues
on the main stream.  ``wait()`` makes the main stream wait for all buckets before the optimizer
runs.  On the NVL backend the buckets live in the symmetric heap and the reduction, the 1/world
scale and any dtype cast are one kernel (``all_reduce_scaled``); on other backends (NCCL, or the
host backend with CPU tensors) it is ``all_reduce`` followed by a scale.

``broadcast_parameters`` makes every rank start from rank 0's weights.  The reference library
offers the primitives this is built from (all_reduce, broadcast: include/megray/communicator.h:86-99)
but no bucketing, overlap or fusion.
"""
from __future__ import annotations

from typing import List

import torch

from ..comm import NVL


class _Bucket:
    def __init__(self, params, flat_w, flat_g):
        self.params = params
        self.flat_w = flat_w
        self.flat_g = flat_g
        self.pending = len(params)
        self.event = None
        self.momentum = None


class GradBucketer:
    def __init__(self, module: torch.nn.Module, comm, bucket_mb: float = 25.0, overlap: bool = True):
        self.comm = comm
        self.world = comm.nranks if comm is not None else 1
        self.overlap = overlap
        params = [p for p in module.parameters() if p.requires_grad]
        if not params:
            raise ValueError("module has no trainable parameters")
        self.cuda = params[0].is_cuda
        self.nvl = comm is not None and comm.backend == NVL and self.cuda
        self.comm_stream = torch.cuda.Stream() if (self.cuda and overlap and comm is not None) else None
        cap = int(bucket_mb * (1 << 20))
        groups, cur, size = [], [], 0
        for p in reversed(params):
            nbytes = p.numel() * p.element_size()
            if cur and (size + nbytes > cap or p.dtype != cur[0].dtype):
                groups.append(cur)
                cur, size = [], 0
            cur.append(p)
            size += nbytes
        if cur:
            groups.append(cur)
        self.buckets: List[_Bucket] = []
        self._bucket_of = {}
        for group in groups:
            numel = sum((p.numel() + 7) // 8 * 8 for p in group)  # 16-byte aligned slots for bf16
            dtype, device = group[0].dtype, group[0].device
            flat_w = torch.empty(numel, dtype=dtype, device=device)
            if self.nvl:
                flat_g = comm.sym_empty((numel,), dtype)
            else:
                flat_g = torch.empty(numel, dtype=dtype, device=device)
            flat_g.zero_()
            off = 0
            for p in group:
                n = p.numel()
                flat_w[off:off + n].copy_(p.data.reshape(-1))
                p.data = flat_w[off:off + n].view(p.shape)
                p.grad = flat_g[off:off + n].view(p.shape)
                off += (n + 7) // 8 * 8
            b = _Bucket(group, flat_w, flat_g)
            self.buckets.append(b)
            for p in group:
                self._bucket_of[p] = b
                p.register_post_accumulate_grad_hook(self._hook)

    # -- backward-time -----------------------------------------------------------------------
    def _hook(self, p: torch.Tensor) -> None:
        b = self._bucket_of[p]
        b.pending -= 1
        if b.pending == 0:
            self._reduce(b)

    def _reduce(self, b: _Bucket) -> None:
        if self.comm is None or self.world == 1:
            return
        scale = 1.0 / self.world
        if self.comm_stream is not None:
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream())
            self.comm_stream.wait_event(ready)
            with torch.cuda.stream(self.comm_stream):
                self._launch(b, scale)
                b.event = torch.cuda.Event()
                b.event.record(self.comm_stream)
        else:
            self._launch(b, scale)

    def _launch(self, b: _Bucket, scale: float) -> None:
        if self.nvl:
            self.comm.all_reduce_scaled(b.flat_g, b.flat_g, scale)
        else:
            self.comm.all_reduce(b.flat_g, b.flat_g, "sum")
            b.flat_g.mul_(scale)

    def wait(self) -> None:
        """All bucket reductions are ordered before whatever the main stream does next."""
        for b in self.buckets:
            if b.pending != 0:
                raise RuntimeError("a gradient bucket is incomplete: some parameter got no gradient")
            if b.event is not None:
                torch.cuda.current_stream().wait_event(b.event)
                b.event = None

    def zero_grad(self) -> None:
        """Gradients accumulate in place into the buckets: clear them before the next backward."""
        for b in self.buckets:
            b.flat_g.zero_()
            b.pending = len(b.params)

    # -- optimizer -----------------------------------------------------------------------------
    def sgd_step(self, lr: float, momentum: float = 0.9, weight_decay: float = 0.0) -> None:
        """One fused SGD(momentum) update per bucket (bf16 CUDA buckets use the library's kernel)."""
        self.wait()
        for b in self.buckets:
            if b.flat_w.is_cuda and b.flat_w.dtype == torch.bfloat16:
                from ..ops import sgd_step as fused_sgd

                if momentum and b.momentum is None:
                    b.momentum = torch.zeros(b.flat_w.numel(), dtype=torch.float32, device=b.flat_w.device)
                fused_sgd(b.flat_w, b.flat_g, lr, b.momentum if momentum else None, momentum, weight_decay)
            else:
                g = b.flat_g if not weight_decay else b.flat_g + weight_decay * b.flat_w
                if momentum:
                    if b.momentum is None:
                        b.momentum = torch.zeros_like(b.flat_w, dtype=torch.float32)
                    b.momentum.mul_(momentum).add_(g.float())
                    b.flat_w.add_(b.momentum.to(b.flat_w.dtype), alpha=-lr)
                else:
                    b.flat_w.add_(g, alpha=-lr)

    def broadcast_parameters(self, root: int = 0) -> None:
        if self.comm is None or self.world == 1:
            return
        for b in self.buckets:
            tmp = torch.empty_like(b.flat_w)
            self.comm.broadcast(b.flat_w, tmp, root)
            b.flat_w.copy_(tmp)

    def bucket_bytes(self) -> List[int]:
        return [b.flat_g.numel() * b.flat_g.element_size() for b in self.buckets]
