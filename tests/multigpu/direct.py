"""Single-pass collectives on symmetric-heap tensors (peer loads/stores, and NVSwitch multimem
when MEGRAY_NVLS=1 and the machine supports multicast) against a CPU reference."""
import os

import torch
from common import setup

rank, n, dev, comm, server = setup()
fails = []


def data(r, numel, dtype, salt=0):
    g = torch.Generator().manual_seed(77 * salt + r)
    if dtype.is_floating_point:
        return (torch.rand(numel, generator=g) * 2 - 1).to(dtype)
    return torch.randint(-100, 100, (numel,), generator=g).to(dtype)


def ref_reduce(xs, op, dtype):
    wide = dtype in (torch.float16, torch.bfloat16)
    acc = xs[0].float() if wide else xs[0].clone()
    for x in xs[1:]:
        x = x.float() if wide else x
        acc = acc + x if op == "sum" else (torch.maximum(acc, x) if op == "max" else torch.minimum(acc, x))
    return acc.to(dtype)


def check(name, got, want, tol=0.0):
    torch.cuda.synchronize()
    g = got.cpu()
    ok = torch.allclose(g.double(), want.double(), rtol=tol, atol=tol) if tol else torch.equal(g, want)
    if not ok:
        fails.append(f"{name} maxdiff={float((g.double() - want.double()).abs().max()):.4g}")


for dtype in (torch.bfloat16, torch.float32, torch.float16, torch.int32):
    for numel in (300_000, (1 << 20) + 24, 5_000_011):
        xs = [data(r, numel, dtype, 1) for r in range(n)]
        a = comm.sym_empty((numel,), dtype)
        b = comm.sym_empty((numel,), dtype)
        a.copy_(xs[rank])
        # bf16/fp16 sums: the switch (or fp32 registers) accumulates in fp32, one rounding at the end;
        # with more than two ranks the order of the fp32 additions may differ from the reference
        # (and the switch's own rounding of 16-bit sums need not be round-to-nearest-even)
        nvls = os.environ.get("MEGRAY_NVLS", "0") == "1"
        tol = 0.0 if ((n == 2 and not nvls) or not dtype.is_floating_point) else 1e-2
        if dtype == torch.float32:
            tol = 1e-5
        for op in ("sum", "max"):
            comm.all_reduce(a, b, op)
            check(f"all_reduce {dtype} {numel} {op}", b, ref_reduce(xs, op, dtype), tol)
        comm.all_reduce(a, a, "sum")  # in place
        check(f"all_reduce in place {dtype} {numel}", a, ref_reduce(xs, "sum", dtype), tol)
        a.copy_(xs[rank])
        m = (numel // n) // 8 * 8
        out = torch.empty(m, dtype=dtype, device=dev)
        comm.reduce_scatter(a[: m * n], out, "sum")
        check(f"reduce_scatter {dtype} {numel}", out, ref_reduce([t[: m * n] for t in xs], "sum", dtype)[rank * m:(rank + 1) * m], tol)
        g = comm.sym_empty((m * n,), dtype)
        comm.all_gather(xs[rank][:m].to(dev), g)
        check(f"all_gather {dtype} {numel}", g, torch.cat([t[:m] for t in xs]))
        comm.all_to_all(xs[rank][: m * n].to(dev), g)  # receive buffer in the heap: direct stores
        check(f"all_to_all {dtype} {numel}", g, torch.cat([xs[q][rank * m:(rank + 1) * m] for q in range(n)]))

# gradient-bucket path: bf16 in, fp32 out, 1/n scale, heap resident
xs = [data(r, 2_000_000, torch.bfloat16, 9) for r in range(n)]
a = comm.sym_empty((2_000_000,), torch.bfloat16)
o = comm.sym_empty((2_000_000,), torch.float32)
a.copy_(xs[rank])
comm.all_reduce_scaled(a, o, 1.0 / n)
check("all_reduce_scaled heap", o, sum(x.float() for x in xs) * (1.0 / n), 1e-2)

st = comm.stats()
assert comm.status == 0 and st["timeouts"] == 0, (comm.status, st)
assert not fails, fails[:8]


def bench(fn, iters=10):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    comm.stream_barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev)
    o = torch.empty_like(t)
    comm.all_reduce(t, o, "max")
    torch.cuda.synchronize()
    return float(o.item())


for nbytes in (1 << 20, 1 << 24, 1 << 28):
    a = comm.sym_empty((nbytes // 2,), torch.bfloat16)
    a.fill_(1.0)
    t = bench(lambda: comm.all_reduce(a, a, "sum"))
    if rank == 0:
        print(f"BW direct all_reduce nvls={os.environ.get('MEGRAY_NVLS', '0')} n={n} bytes={nbytes} time_us={t * 1000:.1f} "
              f"busbw={nbytes / t / 1e6 * 2 * (n - 1) / n:.1f}GB/s", flush=True)
print(f"RANK_OK {rank} nvls_calls={comm.stats()['nvls']} direct_calls={comm.stats()['twoshot']}", flush=True)
comm.close()
