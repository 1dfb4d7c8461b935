"""Tensor-parallel (+ sequence-parallel) SwiGLU MLP stack with explicit forward/backward.

Per layer, with T tokens, model width d, FFN width f and n ranks (f_l = f / n):

    forward    x_n = rmsnorm(x)               on the token shard (fused with the residual add)
               xg  = all_gather(x_n)          [T/n, d] -> [T, d]          (n > 1)
               G|U = xg @ [Wg; Wu]^T          fused epilogue also writes H = silu(G) * U
               yp  = H @ Wd^T                 [T, d] partial sums
               y   = reduce_scatter(yp)       [T, d] -> [T/n, d]          (n > 1);  x <- x + y
    backward   dyg = all_gather(dy)
               dG|dU = (dyg @ Wd) with the SwiGLU derivative fused into the epilogue
               dWd = dyg^T @ H
               dxp = dG|dU @ [Wg; Wu];  dx = reduce_scatter(dxp)
               dWgu = (dG|dU)^T @ xg

Every matrix product runs on the library's tcgen05 kernel (``ops.gemm``); weight and
activation gradients read their operands in transposed storage through TMA, so no
transposition pass exists.  Collectives are the native NVL backend's; with
``fused=True`` the all_gather is overlapped with the GEMM that consumes it and the
reduce_scatter with the GEMM that produces it (``parallel.tensor_parallel``).

The reference library has no model code: this is the tensor-parallel harness that the
library's collectives are built to serve.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from ..ops import (EPI_DSWIGLU, EPI_SWIGLU, add_rmsnorm, gemm, gemm_split_k, mse_loss_grad, pick_split_k,
                   rmsnorm_bwd, sgd_step)


@dataclass
class TPMLPConfig:
    d_model: int = 8192
    ffn: int = 28672
    layers: int = 4
    tokens: int = 8 * 4096      # global tokens per step
    init_std: float = 0.02
    lr: float = 1e-4
    seed: int = 0


class _Layer:
    def __init__(self, cfg: TPMLPConfig, layer: int, rank: int, n: int, device):
        d, f = cfg.d_model, cfg.ffn
        fl = f // n
        g = torch.Generator(device=device).manual_seed(cfg.seed * 1000 + layer)
        # global weights from one seed, then this rank's shard (the same numbers for every n)
        w_gate = torch.empty(f, d, device=device, dtype=torch.bfloat16).normal_(0, cfg.init_std, generator=g)
        w_up = torch.empty(f, d, device=device, dtype=torch.bfloat16).normal_(0, cfg.init_std, generator=g)
        w_down = torch.empty(d, f, device=device, dtype=torch.bfloat16).normal_(0, cfg.init_std, generator=g)
        sl = slice(rank * fl, (rank + 1) * fl)
        self.w_gu = torch.cat([w_gate[sl], w_up[sl]], 0).contiguous()   # [2 f_l, d]
        self.w_down = w_down[:, sl].contiguous()                          # [d, f_l]
        del w_gate, w_up, w_down
        self.g_gu = torch.empty_like(self.w_gu)
        self.g_down = torch.empty_like(self.w_down)
        self.fl = fl


class TPMLPStack:
    """``layers`` pre-norm residual SwiGLU MLP blocks, x <- x + MLP(rmsnorm(x)), sharded over the
    ranks of ``comm`` (None = 1 GPU).  The normalisation (no learnable gain) and the residual
    add are one fused memory-bound kernel between the tensor-parallel regions; they act on the
    token shard, before the all_gather and after the reduce_scatter."""

    def __init__(self, cfg: TPMLPConfig, comm=None, device=None, fused: bool = True):
        self.cfg = cfg
        self.comm = comm
        self.n = comm.nranks if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        if cfg.ffn % (self.n * 128) or cfg.tokens % (self.n * 128) or cfg.d_model % 256:
            raise ValueError("ffn and tokens must be multiples of 128 * nranks, d_model of 256")
        self.layers: List[_Layer] = [_Layer(cfg, l, self.rank, self.n, self.device) for l in range(cfg.layers)]
        T, d, fl, L = cfg.tokens, cfg.d_model, cfg.ffn // self.n, cfg.layers
        self.Ts = T // self.n
        bf = dict(dtype=torch.bfloat16, device=self.device)
        self.tp = None
        if self.n > 1:
            from ..parallel.tensor_parallel import TensorParallelOps

            self.tp = TensorParallelOps(comm, T, d, fused=fused)
        # kept for backward, one set per layer
        self.xg = [self._full(T, d) for _ in range(L)]           # normalised input, all tokens
        self.inv_rms = [torch.empty(self.Ts, dtype=torch.float32, device=self.device) for _ in range(L)]
        self.gu = [torch.empty(T, 2 * fl, **bf) for _ in range(L)]
        self.h = [torch.empty(T, fl, **bf) for _ in range(L)]
        # residual stream and scratch shared by all layers
        self.xs = [torch.empty(self.Ts, d, **bf) for _ in range(2)]
        self.y = torch.empty(self.Ts, d, **bf)
        self.dgu = torch.empty(T, 2 * fl, **bf)
        self.partial = (torch.empty(T, d, **bf) if self.n > 1 and not self.tp.fused else None)
        self.dyg = self._full(T, d) if self.n > 1 else None
        self.dn = torch.empty(self.Ts, d, **bf)
        # gradient of the residual stream: the source of the backward gather, so peers read it
        self.dres = [self.tp.shard_buffer() if self.tp is not None else torch.empty(self.Ts, d, **bf)
                     for _ in range(2)]
        self.dy0 = self.tp.shard_buffer() if self.tp is not None else None
        self.x_dev = torch.empty(self.Ts, d, **bf)
        self._wgrad_ws = None  # partial products of split-K weight-gradient GEMMs

    def _full(self, T, d):
        if self.tp is not None:
            return self.tp.full_buffer()
        return torch.empty(T, d, dtype=torch.bfloat16, device=self.device)

    def _shard(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's rows of an all-token buffer."""
        return full[self.rank * self.Ts:(self.rank + 1) * self.Ts]

    # ------------------------------------------------------------------ forward / backward
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """x: this rank's [T/n, d] token shard (bf16).  Returns the [T/n, d] output shard."""
        L = len(self.layers)
        add_rmsnorm(x, None, None, self._shard(self.xg[0]), self.inv_rms[0])
        for l, layer in enumerate(self.layers):
            fl = layer.fl
            if self.tp is None:
                gemm(self.xg[l], layer.w_gu, self.gu[l], epilogue=EPI_SWIGLU, out2=self.h[l], n=fl)
                gemm(self.h[l], layer.w_down, self.y)
            else:
                self.tp.ag_gemm_swiglu(self.xg[l], layer.w_gu, self.gu[l], self.h[l], fl)
                self.tp.gemm_rs(self.h[l], layer.w_down, self.partial, self.y)
            x_next = self.xs[l & 1]
            if l + 1 < L:
                add_rmsnorm(x, self.y, x_next, self._shard(self.xg[l + 1]), self.inv_rms[l + 1])
            else:
                add_rmsnorm(x, self.y, x_next, None, None)
            x = x_next
        return x

    def backward(self, dy: torch.Tensor) -> torch.Tensor:
        """dy: gradient of the loss w.r.t. the output shard.  Fills the weight gradients and
        returns the gradient w.r.t. the input shard."""
        if self.dy0 is not None and dy is not self.dy0:
            self.dy0.copy_(dy)  # the backward gather reads its source from peers' heaps
            dy = self.dy0
        dres = dy
        for l in reversed(range(len(self.layers))):
            layer = self.layers[l]
            fl = layer.fl
            if self.tp is None:
                gemm(dres, layer.w_down, self.dgu, b_mn=True, epilogue=EPI_DSWIGLU, aux=self.gu[l], n=fl)
                self._wgrad(dres, self.h[l], layer.g_down)
                gemm(self.dgu, layer.w_gu, self.dn, b_mn=True)
                self._wgrad(self.dgu, self.xg[l], layer.g_gu)
            else:
                self.tp.ag_gemm_dswiglu(dres, self.dyg, layer.w_down, self.gu[l], self.dgu, fl)
                self._wgrad(self.dyg, self.h[l], layer.g_down)
                self.tp.gemm_rs(self.dgu, layer.w_gu, self.partial, self.dn, b_mn=True)
                self._wgrad(self.dgu, self.xg[l], layer.g_gu)
            out = self.dres[l & 1]
            rmsnorm_bwd(self.dn, self._shard(self.xg[l]), self.inv_rms[l], dres, out)
            dres = out
        return dres

    def _wgrad(self, a_t: torch.Tensor, b_t: torch.Tensor, out: torch.Tensor) -> None:
        """out[M, N] = a_t^T @ b_t over all tokens (a_t: [T, M], b_t: [T, N]).  The output of a
        sharded layer has few tiles and the token loop is long, so K is cut into the number of
        ranges that fills the waves of CTA pairs best (1 = a plain GEMM)."""
        M, N, K = a_t.shape[1], b_t.shape[1], a_t.shape[0]
        splits = pick_split_k(M, N, K) if out.is_contiguous() else 1
        if splits == 1:
            gemm(a_t, b_t, out, a_mn=True, b_mn=True)
            return
        need = splits * M * N
        if self._wgrad_ws is None or self._wgrad_ws.numel() < need:
            self._wgrad_ws = torch.empty(need, dtype=torch.float32, device=self.device)
        gemm_split_k(a_t, b_t, out, splits, self._wgrad_ws[:need].view(splits * M, N), a_mn=True, b_mn=True)

    def optimizer_step(self) -> None:
        for layer in self.layers:
            sgd_step(layer.w_gu, layer.g_gu, self.cfg.lr)
            sgd_step(layer.w_down, layer.g_down, self.cfg.lr)

    # ------------------------------------------------------------------ public training step
    def train_step_device(self, x: torch.Tensor) -> torch.Tensor:
        """One optimisation step on a device-resident token shard; returns the loss (1-element
        fp32 device tensor: this rank's share of the mean squared output)."""
        y = self.forward(x)
        loss, dy = mse_loss_grad(y, None, 1.0 / (self.cfg.tokens * self.cfg.d_model), dy=self.dy0)
        self.backward(dy)
        self.optimizer_step()
        return loss

    def train_step(self, x_host: torch.Tensor) -> float:
        """The call a user makes: ``x_host`` is this rank's token shard in pinned host memory.
        Copies it to the GPU, runs forward, loss, backward and the SGD update, and returns
        the loss as a Python float (a device-to-host read)."""
        self.x_dev.copy_(x_host, non_blocking=True)
        return float(self.train_step_device(self.x_dev).item())

    def train_step_async(self, x_host: torch.Tensor):
        """Pipelined form of :meth:`train_step` for training loops: the host-to-device copy of
        this step's tokens runs on a copy stream (into one of two device buffers) and the loss
        travels back to pinned host memory asynchronously, so neither transfer stalls the GPU.
        Returns the loss of the PREVIOUS step (None on the first call); :meth:`flush` returns the
        last one.  Every step still copies its own inputs in and its own loss out."""
        if not hasattr(self, "_pipe"):
            self._pipe = {
                "copy": torch.cuda.Stream(), "i": 0,
                "x": [torch.empty_like(self.x_dev) for _ in range(2)],
                "loss": torch.zeros(2, dtype=torch.float32, pin_memory=True),
                "free": [None, None], "done": [None, None],
            }
        p = self._pipe
        k = p["i"] & 1
        main = torch.cuda.current_stream()
        with torch.cuda.stream(p["copy"]):
            if p["free"][k] is not None:
                p["copy"].wait_event(p["free"][k])  # the step that last read this buffer is finished
            p["x"][k].copy_(x_host, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(p["copy"])
        main.wait_event(ready)
        loss = self.train_step_device(p["x"][k])
        p["free"][k] = torch.cuda.Event()
        p["free"][k].record(main)
        p["loss"][k:k + 1].copy_(loss, non_blocking=True)
        p["done"][k] = torch.cuda.Event()
        p["done"][k].record(main)
        p["i"] += 1
        prev = k ^ 1
        if p["done"][prev] is None:
            return None
        p["done"][prev].synchronize()
        return float(p["loss"][prev])

    def flush(self):
        """Loss of the most recent :meth:`train_step_async` call (waits for it)."""
        p = getattr(self, "_pipe", None)
        if p is None or p["i"] == 0:
            return None
        k = (p["i"] - 1) & 1
        p["done"][k].synchronize()
        return float(p["loss"][k])

    def parameters(self):
        for layer in self.layers:
            yield layer.w_gu
            yield layer.w_down

    def flops_per_step(self) -> float:
        """Matrix-multiply FLOPs of one step over all ranks (forward + backward)."""
        c = self.cfg
        return 3 * 6.0 * c.tokens * c.d_model * c.ffn * c.layers
