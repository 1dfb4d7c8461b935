#!/usr/bin/env python
"""Headline benchmark: tensor-parallel transformer MLP training step, tokens/s.

Configuration (the one the baseline names): bf16, d_model 8192, ffn 28672, SwiGLU,
8 x 4096 = 32768 tokens per step ~N(0,1), weights N(0, 0.02), 4 stacked layers, forward +
backward + SGD update, weights sharded over the N GPUs of one node with sequence-parallel
all_gather -> GEMM and GEMM -> reduce_scatter.  Total work is fixed as N grows (strong
scaling).  Synthetic data, random-init weights.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # stock PyTorch GEMMs + the unmodified
                                                             # reference library's NCCL backend

For N > 1 launch one process per GPU (torchrun / python -m torch.distributed.run); when
WORLD_SIZE is absent and --gpus > 1 the script re-launches itself that way.  Rank 0 prints
one JSON line.  `value` is device-timed (CUDA events around exactly K steps, max over
ranks); `e2e` is the same step through the public `TPMLPStack.train_step_async` call, which
every step copies that step's tokens from pinned host memory (on a copy stream) and reads that
step's loss back (asynchronously, delivered one call later), timed on the host clock between
two synchronisations.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--d-model", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--tokens", type=int, default=8 * 4096)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--unfused", action="store_true", help="plain collectives instead of the fused kernels")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--reference", default=None,
                    help="source tree of the reference library (only needed when baseline/_ref is not built yet)")
    return ap.parse_args()


from megray_b200.utils.clocks import ClockSampler  # noqa: E402  (no torch / native code behind it)

METRIC = ("TP-MLP tokens/s (bf16, d_model 8192, ffn 28672, SwiGLU, 32768 tokens, 4 pre-norm residual layers, "
          "fwd+bwd+SGD)")


def config_dict(args, world):
    """The same keys and values in both arms (what differs between them goes under `arm`)."""
    return {"model": f"tp_mlp_d{args.d_model}_f{args.ffn}_L{args.layers}_swiglu", "global_batch": args.tokens,
            "seq_len": 4096, "parallelism": f"tp{world}+sp" if world > 1 else "single",
            "l2": "inputs larger than L2 (weights 1.4 GB/layer, activations > 0.5 GB)"}


def loss_file(args, world):
    """Where the reference arm leaves its loss for this arm to compare with (same box, same
    configuration, same number of steps)."""
    import tempfile

    key = f"n{world}_d{args.d_model}_f{args.ffn}_t{args.tokens}_L{args.layers}_w{args.warmup}_k{args.steps}"
    return os.path.join(tempfile.gettempdir(), f"megray_bench_reference_loss_{key}.json")


def relaunch_multi(args) -> int:
    port = int(os.environ.get("MASTER_PORT", "29533"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)] + sys.argv[1:]
    return subprocess.call(cmd)


# ------------------------------------------------------------------------------------- our arm

def run_ours(args, rank, world, local_rank):
    import torch

    os.environ.setdefault("MEGRAY_HEAP_MB", "6144")
    import megray_b200 as mr
    from megray_b200 import _lib
    from megray_b200.models import TPMLPConfig, TPMLPStack

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    lib = _lib.load(build_if_missing=True)
    comm = None
    server = None
    if world > 1:
        port = int(os.environ.get("MASTER_PORT", "29533")) + 1
        if rank == 0:
            server = mr.Server(world, port)
        comm = mr.Communicator(world, rank, "nvl").init("127.0.0.1", port)

    cfg = TPMLPConfig(d_model=args.d_model, ffn=args.ffn, tokens=args.tokens, layers=args.layers)
    model = TPMLPStack(cfg, comm, dev, fused=not args.unfused)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_dev = torch.randn(cfg.tokens // world, cfg.d_model, device=dev, generator=g).to(torch.bfloat16)
    x_host = torch.empty(x_dev.shape, dtype=torch.bfloat16, pin_memory=True)
    x_host.copy_(x_dev)
    scratch = torch.zeros(4, device=dev, dtype=torch.float32)

    def barrier():
        if comm is not None:
            comm.stream_barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if comm is None:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float32)
        o = torch.empty_like(t)
        comm.all_reduce(t, o, "max")
        torch.cuda.synchronize()
        return float(o.item())

    for _ in range(args.warmup):
        model.train_step_device(x_dev)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = lib.megray_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = model.train_step_device(x_dev)
    e1.record()
    barrier()
    launches = lib.megray_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    # the loss of the whole batch: every rank holds the share of its token shard
    if comm is not None:
        total = torch.empty_like(loss)
        comm.all_reduce(loss, total, "sum")
        torch.cuda.synchronize()
        loss_val = float(total.item())
    else:
        loss_val = float(loss.item())

    e2e = None
    if not args.no_e2e:
        # the public training-loop call: per step one pinned-host -> device copy of the tokens and
        # one device -> host read of the loss, both pipelined with the previous / next step
        model.train_step_async(x_host)
        model.flush()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.train_step_async(x_host)
        model.flush()
        barrier()
        e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1000.0 / args.steps)
        e2e = {"value": cfg.tokens / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": x_host.numel() * x_host.element_size(), "d2h_bytes_per_step": 4}
    from megray_b200.ops import gemm_error_flag

    err = int(gemm_error_flag(dev).item())
    status = comm.status if comm is not None else 0
    if comm is not None:
        comm.close()
    if server is not None:
        server.close()
    if rank != 0:
        return 0
    # Both arms start from the same weights and tokens and take the same number of steps, so
    # their losses must agree to bf16 accuracy.  The reference arm, when it ran before this one on
    # this machine, left its loss in a file.
    loss_check = None
    try:
        with open(loss_file(args, world)) as f:
            ref_loss = float(json.load(f)["loss"])
        rel = abs(loss_val - ref_loss) / max(abs(ref_loss), 1e-12)
        loss_check = {"reference_loss": ref_loss, "rel_diff": rel, "ok": rel < 0.01}
    except (OSError, ValueError, KeyError):
        pass
    out = {
        "metric": METRIC,
        "value": cfg.tokens / (ms / 1000.0), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": config_dict(args, world),
        "arm": {"stack": "tcgen05 GEMM kernels + native NVL collectives of this library",
                "fused_collectives": world > 1 and not args.unfused},
        "tflops_per_gpu": model.flops_per_step() / world / (ms / 1000.0) / 1e12,
        "gpu_launches": int(launches), "clocks": clocks, "e2e": e2e, "loss": loss_val,
        "loss_check": loss_check, "kernel_error_flag": err, "comm_status": status,
    }
    print(json.dumps(out), flush=True)
    if loss_check is not None and not loss_check["ok"]:
        print(f"bench.py: loss {loss_val} differs from the reference arm's {loss_check['reference_loss']} "
              f"by more than 1 %", file=sys.stderr)
        return 1
    return 0 if err == 0 and status == 0 else 1


# ------------------------------------------------------------------------------- reference arm

def run_reference(args, rank, world, local_rank):
    """Stock PyTorch (cuBLAS GEMMs, autograd, torch.optim.SGD) with the collectives of the
    unmodified reference library (its NCCL backend) from baseline/_ref."""
    import ctypes as C

    lib_path = os.path.join(ROOT, "baseline", "_ref", "libmegray_ref.so")
    if not os.path.exists(lib_path):
        try:
            sys.path.insert(0, os.path.join(ROOT, "baseline"))
            import build_ref

            src = args.reference or os.environ.get("MEGRAY_REFERENCE")
            if not src:
                raise RuntimeError("baseline/_ref is not built and neither --reference nor MEGRAY_REFERENCE "
                                   "names the reference source tree")
            build_ref.build(src)
        except Exception as e:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  f"reference library not built ({type(e).__name__}: {str(e)[:120]})"}))
            return 0
    import torch
    import torch.nn.functional as F

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    os.environ.setdefault("NCCL_LAUNCH_MODE", "PARALLEL")
    try:
        ref = C.CDLL(lib_path, mode=C.RTLD_LOCAL)
    except OSError as e:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"cannot load reference library: {str(e)[:150]}"}))
        return 0
    ref.ref_comm_new.restype = C.c_void_p
    ref.ref_comm_init.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
    ref.ref_all_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    ref.ref_reduce_scatter.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    ref.ref_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    port = int(os.environ.get("MASTER_PORT", "29533")) + 2
    if rank == 0:
        assert ref.ref_create_server(world, port) == 0
    comm = ref.ref_comm_new(world, rank)
    assert comm and ref.ref_comm_init(comm, b"127.0.0.1", port) == 0
    FLOAT16, FLOAT32 = 6, 7  # the reference has no bf16 dtype: 2-byte elements travel as float16 bit patterns
                             # for data movement; the reduce_scatter sums them as fp16, so partial sums are
                             # exchanged in fp16 (same byte count as bf16)

    def stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    class AllGather(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            out = torch.empty(world * x.shape[0], x.shape[1], dtype=x.dtype, device=x.device)
            rc = ref.ref_all_gather(comm, x.data_ptr(), out.data_ptr(), x.numel(), FLOAT16, stream())
            assert rc == 0
            return out

        @staticmethod
        def backward(ctx, g):
            g = g.contiguous().to(torch.float16)
            out = torch.empty(g.shape[0] // world, g.shape[1], dtype=torch.float16, device=g.device)
            rc = ref.ref_reduce_scatter(comm, g.data_ptr(), out.data_ptr(), out.numel(), FLOAT16, 0, stream())
            assert rc == 0
            return out.to(torch.bfloat16)

    class ReduceScatter(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            x = x.contiguous().to(torch.float16)
            out = torch.empty(x.shape[0] // world, x.shape[1], dtype=torch.float16, device=x.device)
            rc = ref.ref_reduce_scatter(comm, x.data_ptr(), out.data_ptr(), out.numel(), FLOAT16, 0, stream())
            assert rc == 0
            return out.to(torch.bfloat16)

        @staticmethod
        def backward(ctx, g):
            g = g.contiguous()
            out = torch.empty(world * g.shape[0], g.shape[1], dtype=g.dtype, device=g.device)
            rc = ref.ref_all_gather(comm, g.data_ptr(), out.data_ptr(), g.numel(), FLOAT16, stream())
            assert rc == 0
            return out

    d, f, T, L = args.d_model, args.ffn, args.tokens, args.layers
    fl = f // world
    params = []
    for l in range(L):
        # one globally seeded weight per layer, then this rank's slice: the same numbers as the
        # library arm's model (megray_b200/models/tp_mlp.py) for every number of ranks
        gen = torch.Generator(device=dev).manual_seed(l)
        w_gate = torch.empty(f, d, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        w_up = torch.empty(f, d, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        w_down = torch.empty(d, f, device=dev, dtype=torch.bfloat16).normal_(0, 0.02, generator=gen)
        sl = slice(rank * fl, (rank + 1) * fl)
        w_gu = torch.cat([w_gate[sl], w_up[sl]], 0).contiguous()
        w_dn = w_down[:, sl].contiguous()
        del w_gate, w_up, w_down
        params.append((w_gu.requires_grad_(), w_dn.requires_grad_()))
    torch.cuda.empty_cache()
    opt = torch.optim.SGD([p for pair in params for p in pair], lr=1e-4)
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_dev = torch.randn(T // world, d, device=dev, generator=gen).to(torch.bfloat16)
    x_host = torch.empty(x_dev.shape, dtype=torch.bfloat16, pin_memory=True)
    x_host.copy_(x_dev)

    def step(x):
        h = x
        for w_gu, w_dn in params:
            nrm = F.rms_norm(h, (d,), eps=1e-6)
            xg = AllGather.apply(nrm) if world > 1 else nrm
            gu = xg @ w_gu.t()
            g_, u_ = gu[:, :fl], gu[:, fl:]
            act = F.silu(g_) * u_
            yp = act @ w_dn.t()
            h = h + (ReduceScatter.apply(yp) if world > 1 else yp)
        loss = h.float().pow(2).sum() / (T * d)   # this rank's share of the mean over all tokens
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss.detach()

    def barrier():
        if world > 1:
            t = torch.zeros(1, device=dev)
            ref.ref_all_reduce(comm, t.data_ptr(), t.data_ptr(), 1, FLOAT32, 0, stream())
        torch.cuda.synchronize()

    def over_ranks(v, op):
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float32)
        ref.ref_all_reduce(comm, t.data_ptr(), t.data_ptr(), 1, FLOAT32, op, stream())
        torch.cuda.synchronize()
        return float(t.item())

    for _ in range(args.warmup):
        step(x_dev)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = step(x_dev)
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = over_ranks(e0.elapsed_time(e1) / args.steps, 1)
    loss_val = over_ranks(float(loss.item()), 0)   # sum of the ranks' shares

    # What the fp16 wire format costs this arm: the reference has no bf16, so every reduce_scatter
    # is wrapped in a bf16 -> fp16 cast of its input and an fp16 -> bf16 cast of its result.  Timed
    # on their own here (same tensors, outside the step) so that the share can be read off.
    cast_ms = 0.0
    if world > 1:
        big = torch.empty(T, d, device=dev, dtype=torch.bfloat16).normal_()
        small = torch.empty(T // world, d, device=dev, dtype=torch.float16).normal_()
        for _ in range(2):
            big.to(torch.float16), small.to(torch.bfloat16)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        c0.record()
        for _ in range(5):
            big.to(torch.float16), small.to(torch.bfloat16)
        c1.record()
        torch.cuda.synchronize()
        cast_ms = c0.elapsed_time(c1) / 5 * 2 * L   # one reduce_scatter forward and one backward per layer
        del big, small

    e2e = None
    if not args.no_e2e:
        # the same loop shape as the library arm's train_step_async: this step's tokens are copied
        # from pinned host memory on a copy stream into one of two device buffers, and this step's
        # loss travels back to pinned host memory asynchronously and is read one call later
        copy_stream = torch.cuda.Stream()
        xs = [torch.empty_like(x_dev) for _ in range(2)]
        loss_host = torch.zeros(2, dtype=torch.float32, pin_memory=True)
        free, done = [None, None], [None, None]
        state = {"i": 0}

        def e2e_step():
            k = state["i"] & 1
            main = torch.cuda.current_stream()
            with torch.cuda.stream(copy_stream):
                if free[k] is not None:
                    copy_stream.wait_event(free[k])
                xs[k].copy_(x_host, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(copy_stream)
            main.wait_event(ready)
            lo = step(xs[k])
            free[k] = torch.cuda.Event()
            free[k].record(main)
            loss_host[k:k + 1].copy_(lo.reshape(1), non_blocking=True)
            done[k] = torch.cuda.Event()
            done[k].record(main)
            state["i"] += 1
            if done[k ^ 1] is not None:
                done[k ^ 1].synchronize()
                return float(loss_host[k ^ 1])
            return None

        def e2e_flush():
            k = (state["i"] - 1) & 1
            done[k].synchronize()
            return float(loss_host[k])

        e2e_step()
        e2e_flush()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            e2e_step()
        e2e_flush()
        barrier()
        e2e_ms = over_ranks((time.perf_counter() - t0) * 1000.0 / args.steps, 1)
        e2e = {"value": T / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": x_host.numel() * 2, "d2h_bytes_per_step": 4}
    if rank == 0:
        try:
            with open(loss_file(args, world), "w") as fh:
                json.dump({"loss": loss_val}, fh)
        except OSError:
            pass
        print(json.dumps({
            "metric": METRIC,
            "value": T / (ms / 1000.0), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "reference",
            "config": config_dict(args, world),
            "arm": {"stack": "torch.matmul/autograd/SGD + reference MegRay NCCL backend (fp16 wire format)",
                    "wire_cast_ms_per_step": cast_ms,
                    "value_without_wire_casts": T / (max(ms - cast_ms, 1e-9) / 1000.0)},
            "tflops_per_gpu": 18.0 * T * d * f * L / world / (ms / 1000.0) / 1e12,
            "gpu_launches": 0, "clocks": clocks, "e2e": e2e, "loss": loss_val,
        }), flush=True)
    ref.ref_comm_delete.argtypes = [C.c_void_p]
    ref.ref_comm_delete(comm)
    return 0


def main() -> int:
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and "WORLD_SIZE" not in os.environ:
        return relaunch_multi(args)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world != args.gpus:
        if rank == 0:
            print(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
        return 2
    if args.impl == "reference":
        return run_reference(args, rank, world, local_rank)
    return run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    sys.exit(main())
