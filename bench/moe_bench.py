#!/usr/bin/env python
"""Expert-parallel MoE layer step (forward + backward + SGD), tokens/s: 64 experts, top-2
routing, hidden 4096, expert FFN 14336 (SwiGLU), bf16, 16384 tokens per GPU, experts sharded
evenly over the ranks.

    torchrun --nproc-per-node N bench/moe_bench.py [--impl ours|baseline] [--steps 5 --warmup 3]

`--impl ours`: megray_b200.models.MoELayer: routing, plan, dispatch and combine kernels fused with
the all-to-all-v over NVLink peer memory, grouped tcgen05 GEMMs, explicit backward.
`--impl baseline`: the composition a user of the reference library writes around its
equal-chunk all_to_all (the unmodified reference from baseline/_ref, NCCL backend): PyTorch routing
(top-2, sort by expert), chunks padded to a fixed capacity, grouped GEMMs for the experts
(torch grouped_mm), index_add combine, autograd backward, torch.optim.SGD.

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


def load_reference():
    """The unmodified reference library (baseline/_ref, built by baseline/build_ref.py), or None."""
    import ctypes as C

    path = os.path.join(ROOT, "baseline", "_ref", "libmegray_ref.so")
    if not os.path.exists(path):
        return None
    os.environ.setdefault("NCCL_LAUNCH_MODE", "PARALLEL")
    ref = C.CDLL(path, mode=C.RTLD_LOCAL)
    ref.ref_comm_new.restype = C.c_void_p
    ref.ref_comm_init.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    ref.ref_all_to_all.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    ref.ref_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    ref.ref_comm_delete.argtypes = [C.c_void_p]
    return ref


def run_baseline(a):
    """What a user of the reference library writes: its all_to_all moves equal chunks only
    (reference include/megray/communicator.h:75-77), so every rank pads what it sends to each peer
    to a fixed capacity (1.25 x the mean, rows beyond it are dropped, as in this library's arm),
    routes and permutes with PyTorch ops, runs the experts as grouped cuBLAS / CUTLASS GEMMs
    (torch grouped_mm; a loop of matmuls where that is unavailable), and lets autograd do the
    backward (the transposed all_to_all is again the reference's call)."""
    import ctypes as C

    import torch.nn.functional as F

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    ref = load_reference()
    comm = None
    if world > 1:
        if ref is None:
            raise SystemExit("baseline/_ref/libmegray_ref.so is missing: run baseline/build_ref.py first")
        port = int(os.environ.get("MASTER_PORT", "29533")) + 7
        if rank == 0:
            assert ref.ref_create_server(world, port) == 0
        comm = ref.ref_comm_new(world, rank)
        assert comm and ref.ref_comm_init(comm, b"127.0.0.1", port) == 0
    FLOAT16, FLOAT32, INT32 = 6, 7, 2
    E, H, Fd, T = a.experts, a.hidden, a.ffn, a.tokens
    El = E // world
    cap = (int(2 * T / world * 1.25) + 127) // 128 * 128   # rows per (source, destination) pair
    w_gu = torch.empty(El, 2 * Fd, H, device=dev, dtype=torch.bfloat16)
    w_dn = torch.empty(El, H, Fd, device=dev, dtype=torch.bfloat16)
    for le in range(El):
        g = torch.Generator(device=dev).manual_seed(rank * El + le)   # the same weights as the library arm
        w_gu[le].normal_(0, 0.02, generator=g)
        w_dn[le].normal_(0, 0.02, generator=g)
    w_gu.requires_grad_()
    w_dn.requires_grad_()
    opt = torch.optim.SGD([w_gu, w_dn], lr=1e-4)
    x, logits = inputs(a, rank, dev)
    x.requires_grad_()
    logits.requires_grad_()

    def stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def a2a_raw(t, dtype_code):
        if world == 1:
            return t.clone()
        out = torch.empty_like(t)
        rc = ref.ref_all_to_all(comm, t.data_ptr(), out.data_ptr(), t.numel() // world, dtype_code, stream())
        assert rc == 0
        return out

    class AllToAll(torch.autograd.Function):   # [world, cap, H] bf16, chunk q goes to rank q
        @staticmethod
        def forward(ctx, t):
            return a2a_raw(t.contiguous(), FLOAT16)   # 2-byte elements: pure data movement

        @staticmethod
        def backward(ctx, g):
            return a2a_raw(g.contiguous(), FLOAT16)

    state = {"grouped": hasattr(F, "grouped_mm")}

    def experts(xs, offs, per_expert):
        if state["grouped"]:
            try:
                gu = F.grouped_mm(xs, w_gu.transpose(-2, -1), offs=offs)
                h = F.silu(gu[:, :Fd]) * gu[:, Fd:]
                return F.grouped_mm(h, w_dn.transpose(-2, -1), offs=offs)
            except (RuntimeError, NotImplementedError):
                state["grouped"] = False
        ys = []
        for le, xe in enumerate(torch.split(xs, per_expert)):
            gu = xe @ w_gu[le].t()
            ys.append((F.silu(gu[:, :Fd]) * gu[:, Fd:]) @ w_dn[le].t())
        return torch.cat(ys)

    def step():
        opt.zero_grad(set_to_none=True)
        x.grad = logits.grad = None
        top, idx = logits.topk(2, dim=-1)                     # the library arm's routing: softmax over the pair
        w = torch.softmax(top, dim=-1)
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)            # (token, slot) pairs by expert, hence by owner
        se = flat_e[order]
        dest = se // El
        first = torch.searchsorted(dest, torch.arange(world, device=dev))
        slot = torch.arange(2 * T, device=dev) - first[dest]  # position inside the chunk for that owner
        keep = slot < cap
        o_k, d_k, s_k = order[keep], dest[keep], slot[keep]
        flat = d_k * cap + s_k
        send = torch.zeros(world * cap, H, device=dev, dtype=torch.bfloat16).index_copy(0, flat, x[o_k // 2])
        ids = torch.full((world * cap,), -1, device=dev, dtype=torch.int32)
        ids[flat] = (se[keep] % El).to(torch.int32)
        recv = AllToAll.apply(send.view(world, cap, H)).view(world * cap, H)
        rid = a2a_raw(ids.view(world, cap), INT32).view(-1).long()
        valid = rid >= 0
        order2 = torch.argsort(torch.where(valid, rid, torch.full_like(rid, El)), stable=True)
        nvalid = valid.sum()
        counts = torch.bincount(rid[valid], minlength=El)
        offs = torch.cumsum(counts, 0).to(torch.int32)
        if state["grouped"]:
            # padding rows are sorted to the end and lie beyond offs[-1]: the grouped GEMM ignores them
            xs = recv[order2]
            ys = experts(xs, offs, None)
        else:
            nv = int(nvalid)                                   # (host read: sizes of the per-expert matmuls)
            xs = recv[order2[:nv]]
            ys = experts(xs, offs, [int(c) for c in counts])
            ys = torch.cat([ys, torch.zeros(world * cap - nv, H, device=dev, dtype=ys.dtype)])
        back_in = torch.zeros(world * cap, H, device=dev, dtype=torch.bfloat16).index_copy(0, order2, ys)
        back = AllToAll.apply(back_in.view(world, cap, H)).view(world * cap, H)
        gate = w.reshape(-1)[o_k].to(torch.bfloat16)
        out = torch.zeros(T, H, device=dev, dtype=torch.bfloat16).index_add(0, o_k // 2, back[flat] * gate[:, None])
        loss = (out.float() ** 2).sum() / (T * world * H)
        loss.backward()
        opt.step()
        return loss.detach()

    def barrier():
        if world > 1:
            t = torch.zeros(1, device=dev)
            ref.ref_all_reduce(comm, t.data_ptr(), t.data_ptr(), 1, FLOAT32, 0, stream())
        torch.cuda.synchronize()

    for _ in range(a.warmup):
        loss = step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    barrier()
    ms = torch.tensor([e0.elapsed_time(e1) / a.steps], device=dev)
    total = loss.reshape(1).float().clone()
    if world > 1:
        ref.ref_all_reduce(comm, ms.data_ptr(), ms.data_ptr(), 1, FLOAT32, 1, stream())
        torch.cuda.synchronize()
    flops = 3 * 6.0 * T * 2 * H * Fd
    out = (rank, world, float(ms.item()), float(total.item()), flops)
    if comm:
        ref.ref_comm_delete(comm)
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
