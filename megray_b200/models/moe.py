"""Expert-parallel mixture-of-experts layer with explicit forward / backward.

Configuration of the MoE benchmark: 64 experts, top-2 routing, hidden 4096, expert FFN 14336
(SwiGLU), bf16, 16384 tokens per GPU, experts sharded evenly over the ranks.

    forward    route -> plan -> dispatch (fused permute + all-to-all) -> grouped SwiGLU GEMM ->
               grouped down GEMM -> combine (fused all-to-all + un-permute + gate-weighted sum)
    backward   gate gradients; dispatch of gate-weighted output gradients; grouped GEMMs for
               dH (with the SwiGLU derivative fused), the two weight gradients (one K range per
               expert) and dX; combine without gates

All matrix products are the library's tcgen05 kernel in its grouped forms: 128-row blocks of
the expert-sorted buffer pick their expert's weights, and weight gradients take one contiguous
row range per expert.  The reference library has no model code.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import EPI_DSWIGLU, EPI_SWIGLU, gemm, mse_loss_grad, sgd_step
from ..parallel.expert_parallel import ExpertParallelOps


@dataclass
class MoEConfig:
    experts: int = 64
    hidden: int = 4096
    ffn: int = 14336
    tokens: int = 16384          # per GPU
    init_std: float = 0.02
    lr: float = 1e-4
    capacity_factor: float = 1.25
    seed: int = 0


class MoELayer:
    def __init__(self, cfg: MoEConfig, comm=None, device=None):
        self.cfg, self.comm = cfg, comm
        self.n = comm.nranks if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        H, F, T = cfg.hidden, cfg.ffn, cfg.tokens
        if H % 256 or F % 128:
            raise ValueError("hidden must be a multiple of 256 and ffn of 128")
        self.ep = ExpertParallelOps(comm, T, H, cfg.experts, cfg.capacity_factor)
        El, cap = self.ep.El, self.ep.capacity
        bf = dict(dtype=torch.bfloat16, device=self.device)
        # expert weights: expert e of this rank is global expert rank*El + e, seeded by its global id
        self.w_gu = torch.empty(El * 2 * F, H, **bf)
        self.w_down = torch.empty(El * H, F, **bf)
        for le in range(El):
            g = torch.Generator(device=self.device).manual_seed(cfg.seed * 100003 + self.rank * El + le)
            self.w_gu[le * 2 * F:(le + 1) * 2 * F].normal_(0, cfg.init_std, generator=g)
            self.w_down[le * H:(le + 1) * H].normal_(0, cfg.init_std, generator=g)
        self.g_gu = torch.empty_like(self.w_gu)
        self.g_down = torch.empty_like(self.w_down)
        # buffers peers write into / read from
        self.x_perm = self.ep.exchange_buffer()
        self.y_perm = self.ep.exchange_buffer()
        self.dy_perm = self.ep.exchange_buffer()
        self.dx_perm = self.ep.exchange_buffer()
        if comm is not None:
            torch.cuda.synchronize()
            comm.stream_barrier()
        self.gu = torch.empty(cap, 2 * F, **bf)
        self.h = torch.empty(cap, F, **bf)
        self.dgu = torch.empty(cap, 2 * F, **bf)
        self.out = torch.empty(T, H, **bf)
        self.dx = torch.empty(T, H, **bf)
        self.dw = torch.empty(T, 2, dtype=torch.float32, device=self.device)
        self.dlogits = torch.empty(T, cfg.experts, dtype=torch.float32, device=self.device)
        self.x_dev = torch.empty(T, H, **bf)
        self.logits_dev = torch.empty(T, cfg.experts, dtype=torch.float32, device=self.device)

    # ------------------------------------------------------------------ forward / backward
    def forward(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        ep, F, H = self.ep, self.cfg.ffn, self.cfg.hidden
        ep.route(logits)
        ep.plan()
        ep.zero_pads(self.x_perm)
        ep.dispatch(x, self.x_perm, first=True)
        ep.barrier()
        grp = dict(m_block_group=ep.block_group, groups=ep.El)
        gemm(self.x_perm, self.w_gu, self.gu, epilogue=EPI_SWIGLU, out2=self.h, n=F, group_rows_b=2 * F, **grp)
        gemm(self.h, self.w_down, self.y_perm, n=H, group_rows_b=H, **grp)
        ep.barrier()
        ep.combine(self.out, self.y_perm, weights=True)
        return self.out

    def backward(self, dout: torch.Tensor):
        """Returns (dx, dlogits); fills the expert weight gradients."""
        ep, F, H = self.ep, self.cfg.ffn, self.cfg.hidden
        ep.combine_dw(dout, self.y_perm, self.dw)
        ep.zero_pads(self.dy_perm)
        ep.dispatch(dout, self.dy_perm, weights=True, first=False)
        ep.barrier()
        grp = dict(m_block_group=ep.block_group, groups=ep.El)
        rng = dict(k_begin=ep.seg_begin, k_end=ep.seg_end, groups=ep.El)
        gemm(self.dy_perm, self.w_down, self.dgu, b_mn=True, epilogue=EPI_DSWIGLU, aux=self.gu, n=F,
             group_rows_b=H, **grp)
        gemm(self.dy_perm, self.h, self.g_down, a_mn=True, b_mn=True, **rng)
        gemm(self.dgu, self.w_gu, self.dx_perm, b_mn=True, n=H, group_rows_b=2 * F, **grp)
        gemm(self.dgu, self.x_perm, self.g_gu, a_mn=True, b_mn=True, **rng)
        ep.barrier()
        ep.combine(self.dx, self.dx_perm, weights=False)
        ep.route_bwd(self.dw, self.dlogits)
        return self.dx, self.dlogits

    def optimizer_step(self) -> None:
        sgd_step(self.w_gu, self.g_gu, self.cfg.lr)
        sgd_step(self.w_down, self.g_down, self.cfg.lr)

    def train_step_device(self, x: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        y = self.forward(x, logits)
        loss, dy = mse_loss_grad(y, None, 1.0 / (self.cfg.tokens * self.n * self.cfg.hidden))
        self.backward(dy)
        self.optimizer_step()
        return loss

    def train_step(self, x_host: torch.Tensor, logits_host: torch.Tensor) -> float:
        """Public call: tokens and router logits come from pinned host memory, the loss goes back."""
        self.x_dev.copy_(x_host, non_blocking=True)
        self.logits_dev.copy_(logits_host, non_blocking=True)
        return float(self.train_step_device(self.x_dev, self.logits_dev).item())

    def flops_per_step(self) -> float:
        """Matrix-multiply FLOPs of one step on this rank's tokens (forward + backward)."""
        c = self.cfg
        return 3 * 6.0 * c.tokens * 2 * c.hidden * c.ffn
