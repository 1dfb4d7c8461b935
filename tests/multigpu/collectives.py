"""Every NVL collective against a CPU reference (run under torchrun)."""
import torch
from common import setup

rank, n, dev, comm, server = setup()


def data(r, numel, dtype, salt=0):
    g = torch.Generator().manual_seed(1000 * salt + r)
    if dtype.is_floating_point:
        return (torch.rand(numel, generator=g) * 2 - 1).to(dtype)
    return torch.randint(-100 if dtype != torch.uint8 else 0, 100, (numel,), generator=g).to(dtype)


def ref_reduce(xs, op, dtype):
    wide = dtype in (torch.float16, torch.bfloat16)
    acc = xs[0].float() if wide else xs[0].clone()
    for x in xs[1:]:
        x = x.float() if wide else x
        acc = acc + x if op == "sum" else (torch.maximum(acc, x) if op == "max" else torch.minimum(acc, x))
    return acc.to(dtype)


fails = []


def check(name, got, want, tol=0.0):
    torch.cuda.synchronize()
    g = got.cpu()
    ok = torch.allclose(g.double(), want.double(), rtol=tol, atol=tol) if tol else torch.equal(g, want)
    if not ok:
        fails.append(name)


dtypes = [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int8, torch.uint8, torch.int64,
          torch.float64]
sizes = [1, 7, 1000, 4099, 65536 + 3, (1 << 20) + 5]
for dtype in dtypes:
    for numel in sizes:
        if dtype not in (torch.float32, torch.bfloat16) and numel > 70000:
            continue
        xs = [data(r, numel, dtype) for r in range(n)]
        x = xs[rank].to(dev)
        tol = 1e-5 if dtype in (torch.float32, torch.float64) else 0.0
        for op in ("sum", "max", "min"):
            out = torch.empty_like(x)
            comm.all_reduce(x, out, op)
            check(f"all_reduce {dtype} {numel} {op}", out, ref_reduce(xs, op, dtype), tol)
        m = numel // n
        root = 1 % n
        if m > 0:
            out = torch.empty(m, dtype=dtype, device=dev)
            comm.reduce_scatter(x[: m * n].contiguous(), out, "sum")
            full = ref_reduce([t[: m * n] for t in xs], "sum", dtype)
            check(f"reduce_scatter {dtype} {numel}", out, full[rank * m:(rank + 1) * m], tol)
            out = torch.empty(m * n, dtype=dtype, device=dev)
            comm.all_to_all(x[: m * n].contiguous(), out)
            check(f"all_to_all {dtype} {numel}", out, torch.cat([xs[q][rank * m:(rank + 1) * m] for q in range(n)]))
            out = torch.empty(m, dtype=dtype, device=dev)
            comm.scatter(x[: m * n].contiguous() if rank == root else None, out, root)
            check(f"scatter {dtype} {numel}", out, xs[root][rank * m:(rank + 1) * m])
        out = torch.empty(n * numel, dtype=dtype, device=dev)
        comm.all_gather(x, out)
        check(f"all_gather {dtype} {numel}", out, torch.cat(xs))
        out = torch.empty_like(x)
        comm.broadcast(x, out, root)
        check(f"broadcast {dtype} {numel}", out, xs[root])
        out = torch.full_like(x, 3)
        comm.reduce(x, out, root, "sum")
        if rank == root:
            check(f"reduce {dtype} {numel}", out, ref_reduce(xs, "sum", dtype), tol)
        out = torch.empty(n * numel, dtype=dtype, device=dev) if rank == root else None
        comm.gather(x, out, root)
        if rank == root:
            check(f"gather {dtype} {numel}", out, torch.cat(xs))

# fused scale + cast (gradient-bucket path)
xs = [data(r, 100003, torch.bfloat16, 5) for r in range(n)]
out = torch.empty(100003, dtype=torch.float32, device=dev)
comm.all_reduce_scaled(xs[rank].to(dev), out, 1.0 / n)
check("all_reduce_scaled bf16->f32", out, sum(x.float() for x in xs) * (1.0 / n), 1e-6)

# buffers inside the symmetric heap work like any others
t = comm.sym_empty((4096,), torch.float32)
t.fill_(rank + 1.0)
o = torch.empty_like(t)
comm.all_reduce(t, o)
check("all_reduce heap tensor", o, torch.full((4096,), n * (n + 1) / 2.0))

# send / recv (NCCL point-to-point engine), grouped so that both directions overlap
a = torch.full((1000,), float(rank), device=dev)
b = torch.empty_like(a)
peer = rank ^ 1
if peer < n:
    comm.group_start()
    comm.send(a, peer)
    comm.recv(b, peer)
    comm.group_end()
    check("send/recv", b, torch.full((1000,), float(peer)))

st = comm.stats()
assert st["timeouts"] == 0 and comm.status == 0, (st, comm.status)
assert not fails, fails[:10]
print(f"RANK_OK {rank} kernels={st['kernels']}", flush=True)
comm.close()
