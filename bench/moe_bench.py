#!/usr/bin/env python
"""Expert-parallel MoE layer step (forward + backward + SGD), tokens/s: 64 experts, top-2
routing, hidden 4096, expert FFN 14336 (SwiGLU), bf16, 16384 tokens per GPU, experts sharded
evenly over the ranks.

    torchrun --nproc-per-node N bench/moe_bench.py [--impl ours|baseline] [--steps 5 --warmup 3]

`--impl ours`: megray_b200.models.MoELayer: routing, plan, dispatch and combine kernels fused with
the all-to-all-v over NVLink peer memory, grouped tcgen05 GEMMs, explicit backward.
`--impl baseline`: the composition a user of the reference library would write around its
equal-chunk all_to_all: PyTorch routing (softmax, top-2, sort by expert), counts exchanged on the
host, NCCL all_to_all (torch.distributed, one NCCL call like the reference's NCCL backend), one
cuBLAS GEMM per expert, index_add combine, autograd backward, torch.optim.SGD.

Device-timed with CUDA events around the timed steps, max over ranks; synthetic seeded data
(tokens ~N(0,1), router logits ~N(0,1)); rank 0 prints one JSON line.  Inputs exceed L2
(expert weights alone are 2.8 GB per GPU at 8 ranks).
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", default="ours", choices=["ours", "baseline"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--tokens", type=int, default=16384, help="per GPU")
    return ap.parse_args()


def inputs(a, rank, dev):
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn(a.tokens, a.hidden, device=dev, generator=g).to(torch.bfloat16)
    logits = torch.randn(a.tokens, a.experts, device=dev, generator=g)
    return x, logits


def run_ours(a):
    from megray_b200.models import MoEConfig, MoELayer
    from megray_b200.ops import gemm_error_flag
    from megray_b200.utils import init_from_env, max_over_ranks

    os.environ.setdefault("MEGRAY_HEAP_MB", "8192")
    rank, world, dev, comm, server = init_from_env()
    cfg = MoEConfig(experts=a.experts, hidden=a.hidden, ffn=a.ffn, tokens=a.tokens)
    layer = MoELayer(cfg, comm, dev)
    x, logits = inputs(a, rank, dev)
    for _ in range(a.warmup):
        loss = layer.train_step_device(x, logits)
    torch.cuda.synchronize()
    if comm is not None:
        comm.stream_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = layer.train_step_device(x, logits)
    e1.record()
    torch.cuda.synchronize()
    ms = max_over_ranks(comm, e0.elapsed_time(e1) / a.steps, dev)
    assert int(gemm_error_flag(dev).item()) == 0
    flops = layer.flops_per_step()
    out = (rank, world, ms, float(loss.item()), flops)
    if comm is not None:
        comm.close()
    return out


def run_baseline(a):
    import torch.distributed as dist
    import torch.nn.functional as F

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    E, H, Fd, T = a.experts, a.hidden, a.ffn, a.tokens
    El = E // world
    w_gu, w_dn = [], []
    for le in range(El):
        g = torch.Generator(device=dev).manual_seed(rank * El + le)
        w_gu.append(torch.empty(2 * Fd, H, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=g).requires_grad_())
        w_dn.append(torch.empty(H, Fd, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=g).requires_grad_())
    opt = torch.optim.SGD(w_gu + w_dn, lr=1e-4)
    x, logits = inputs(a, rank, dev)
    x.requires_grad_()
    logits.requires_grad_()

    class AllToAll(torch.autograd.Function):
        @staticmethod
        def forward(ctx, t, out_splits, in_splits):
            ctx.splits = (out_splits, in_splits)
            if world == 1:
                return t.clone()
            out = t.new_empty(sum(out_splits), t.shape[1])
            dist.all_to_all_single(out, t.contiguous(), out_splits, in_splits)
            return out

        @staticmethod
        def backward(ctx, g):
            out_splits, in_splits = ctx.splits
            if world == 1:
                return g.clone(), None, None
            out = g.new_empty(sum(in_splits), g.shape[1])
            dist.all_to_all_single(out, g.contiguous(), in_splits, out_splits)
            return out, None, None

    def step():
        opt.zero_grad(set_to_none=True)
        x.grad = logits.grad = None
        probs = torch.softmax(logits, dim=-1)
        w, idx = probs.topk(2, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        tok = order // 2
        counts = torch.bincount(flat_e, minlength=E)
        # counts travel through the host, as they must with an equal-chunk / split-list all_to_all
        if world > 1:
            counts_all = torch.empty(world, E, dtype=counts.dtype, device=dev)
            dist.all_gather_into_tensor(counts_all, counts)
        else:
            counts_all = counts[None]
        ca = counts_all.cpu()
        in_splits = [int(ca[rank, q * El:(q + 1) * El].sum()) for q in range(world)]
        out_splits = [int(ca[q, rank * El:(rank + 1) * El].sum()) for q in range(world)]
        recv = AllToAll.apply(x[tok], out_splits, in_splits)
        # received rows are grouped by source rank, then by local expert: regroup by expert
        mine = ca[:, rank * El:(rank + 1) * El]  # [world, El]
        eid = torch.repeat_interleave(torch.arange(El).repeat(world), mine.reshape(-1)).to(dev)
        order2 = torch.argsort(eid, stable=True)
        xs = recv[order2]
        per_expert = [int(v) for v in mine.sum(0)]
        ys = []
        for le, xe in enumerate(torch.split(xs, per_expert)):
            if xe.shape[0] == 0:
                continue
            gu = xe @ w_gu[le].t()
            h = F.silu(gu[:, :Fd]) * gu[:, Fd:]
            ys.append(h @ w_dn[le].t())
        outs = torch.empty_like(xs).index_copy(0, order2, torch.cat(ys))
        back = AllToAll.apply(outs, in_splits, out_splits)
        gate = w.reshape(-1)[order].to(torch.bfloat16)
        out = torch.zeros(T, H, device=dev, dtype=torch.bfloat16).index_add(0, tok, back * gate[:, None])
        loss = (out.float() ** 2).sum() / (T * world * H)
        loss.backward()
        opt.step()
        return loss

    for _ in range(a.warmup):
        loss = step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    flops = 3 * 6.0 * T * 2 * H * Fd
    out = (rank, world, float(ms.item()), float(loss.item()), flops)
    if world > 1:
        dist.destroy_process_group()
    return out


def main():
    a = parse()
    rank, world, ms, loss, flops = run_ours(a) if a.impl == "ours" else run_baseline(a)
    if rank == 0:
        print(json.dumps({
            "metric": "MoE layer tokens/s (64 experts, top-2, hidden 4096, ffn 14336, bf16, fwd+bwd+SGD)",
            "impl": a.impl, "value": a.tokens * world / ms * 1e3, "unit": "tokens/s", "n_gpus": world,
            "ms_per_step": ms, "steps": a.steps, "warmup": a.warmup, "loss": loss,
            "tflops_per_gpu": flops / ms / 1e9, "tokens_per_gpu": a.tokens, "data": "synthetic"}), flush=True)


if __name__ == "__main__":
    main()
