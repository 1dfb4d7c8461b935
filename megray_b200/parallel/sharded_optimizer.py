"""Data parallelism with the optimizer state sharded over the ranks (ZeRO stage 1).

All parameters live in one flat buffer (every ``p.data`` is a view into it) and all gradients in
another.  A step is: reduce_scatter of the flat gradient (each rank receives the mean of its own
1/world slice), SGD with momentum on that slice only (so the momentum costs 1/world of the
parameter count per rank), all_gather of the updated slices back into every rank's flat parameter
buffer.  The two collectives move the same bytes as the all_reduce they replace.

Built on reduce_scatter and all_gather (include/megray/communicator.h:79-95 in the reference,
which has no optimizer code); works with CUDA tensors on the NVL / NCCL backends and with CPU
tensors on the host backend.
"""
from __future__ import annotations

import torch


class ShardedSGD:
    def __init__(self, module: torch.nn.Module, comm, lr: float, momentum: float = 0.9, weight_decay: float = 0.0):
        self.comm, self.lr, self.mu, self.wd = comm, lr, momentum, weight_decay
        self.world = comm.nranks if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.params = [p for p in module.parameters() if p.requires_grad]
        if not self.params:
            raise ValueError("module has no trainable parameters")
        dtype, device = self.params[0].dtype, self.params[0].device
        if any(p.dtype != dtype or p.device != device for p in self.params):
            raise ValueError("all parameters must share one dtype and device")
        total = sum(p.numel() for p in self.params)
        # every rank's slice has the same length, a multiple of 8 elements (16-byte vectors)
        self.shard = -(-total // (self.world * 8)) * 8
        self.flat_w = torch.zeros(self.shard * self.world, dtype=dtype, device=device)
        self.flat_g = torch.zeros_like(self.flat_w)
        off = 0
        for p in self.params:
            n = p.numel()
            self.flat_w[off:off + n].copy_(p.data.reshape(-1))
            p.data = self.flat_w[off:off + n].view_as(p)
            p.grad = self.flat_g[off:off + n].view_as(p)
            off += n
        self.g_shard = torch.empty(self.shard, dtype=dtype, device=device)
        # arithmetic and momentum in fp32 for 16-bit parameters, else in the parameters' own type
        self.acc = torch.float32 if dtype in (torch.float16, torch.bfloat16) else dtype
        self.momentum = torch.zeros(self.shard, dtype=self.acc, device=device) if momentum else None

    def my_slice(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.rank * self.shard:(self.rank + 1) * self.shard]

    def zero_grad(self) -> None:
        self.flat_g.zero_()

    def broadcast_parameters(self, root: int = 0) -> None:
        """Every rank starts from ``root``'s weights."""
        if self.comm is not None and self.world > 1:
            self.comm.broadcast(self.flat_w, self.flat_w, root)

    def state_bytes_per_rank(self) -> int:
        """Optimizer state held by this rank (the point of the sharding)."""
        return 0 if self.momentum is None else self.momentum.numel() * self.momentum.element_size()

    @torch.no_grad()
    def step(self) -> None:
        if self.comm is not None and self.world > 1:
            self.comm.reduce_scatter(self.flat_g, self.g_shard, "sum")
            g = self.g_shard.to(self.acc) / self.world
        else:
            g = self.flat_g.to(self.acc)
        w = self.my_slice(self.flat_w)
        wf = w.to(self.acc)
        if self.wd:
            g = g + self.wd * wf
        if self.momentum is not None:
            self.momentum.mul_(self.mu).add_(g)
            g = self.momentum
        w.copy_((wf - self.lr * g).to(w.dtype))
        if self.comm is not None and self.world > 1:
            # in place: slice r of the flat buffer is rank r's contribution
            self.comm.all_gather(w.clone(), self.flat_w)
