"""Single-pass collectives on ordinary CUDA tensors registered with the communicator (one process
per GPU: peers map the buffers through CUDA IPC handles), against a CPU reference, next to the
staged path on the same data before registration and after deregistration."""
import torch
from common import setup

rank, n, dev, comm, server = setup()
fails = []


def data(r, numel, dtype, salt=0):
    g = torch.Generator().manual_seed(131 * salt + r)
    if dtype.is_floating_point:
        return (torch.rand(numel, generator=g) * 2 - 1).to(dtype)
    return torch.randint(-100, 100, (numel,), generator=g).to(dtype)


def ref_sum(xs, dtype):
    wide = dtype in (torch.float16, torch.bfloat16)
    acc = xs[0].float() if wide else xs[0].clone()
    for x in xs[1:]:
        acc = acc + (x.float() if wide else x)
    return acc.to(dtype)


def check(name, got, want, tol=0.0):
    torch.cuda.synchronize()
    g = got.cpu()
    ok = torch.allclose(g.double(), want.double(), rtol=tol, atol=tol) if tol else torch.equal(g, want)
    if not ok:
        fails.append(f"{name} maxdiff={float((g.double() - want.double()).abs().max()):.4g}")


for dtype in (torch.bfloat16, torch.float32, torch.int32):
    numel = (1 << 20) + 24
    xs = [data(r, numel, dtype, 3) for r in range(n)]
    tol = 0.0 if (n == 2 or not dtype.is_floating_point) else (1e-5 if dtype == torch.float32 else 1e-2)
    m = (numel // n) // 8 * 8
    # separate allocations (not slices of one caching-allocator block would also work)
    a = torch.empty(numel, dtype=dtype, device=dev)
    b = torch.empty(numel, dtype=dtype, device=dev)
    g = torch.empty(m * n, dtype=dtype, device=dev)
    a.copy_(xs[rank])
    want = ref_sum(xs, dtype)

    comm.all_reduce(a, b, "sum")  # staged: nothing registered yet
    check(f"staged all_reduce {dtype}", b, want, tol)

    shared = comm.register(a) and comm.register(b) and comm.register(g)
    assert shared, "cudaMalloc memory must be shareable between processes"
    b.zero_()
    comm.all_reduce(a, b, "sum")
    check(f"registered all_reduce {dtype}", b, want, tol)
    comm.all_reduce(a, a, "sum")  # in place
    check(f"registered all_reduce in place {dtype}", a, want, tol)
    a.copy_(xs[rank])
    out = torch.empty(m, dtype=dtype, device=dev)
    comm.reduce_scatter(a[: m * n], out, "sum")
    check(f"registered reduce_scatter {dtype}", out, ref_sum([t[: m * n] for t in xs], dtype)[rank * m:(rank + 1) * m], tol)
    comm.all_gather(xs[rank][:m].to(dev), g)
    check(f"registered all_gather {dtype}", g, torch.cat([t[:m] for t in xs]))
    comm.all_to_all(xs[rank][: m * n].to(dev), g)
    check(f"registered all_to_all {dtype}", g, torch.cat([xs[q][rank * m:(rank + 1) * m] for q in range(n)]))
    # a view at the same distance from the start on every rank qualifies too
    half = (numel // 2) // 8 * 8
    comm.all_reduce(a[half:], b[half:], "sum")
    check(f"registered all_reduce on a view {dtype}", b[half:], ref_sum([t[half:] for t in xs], dtype), tol)

    comm.deregister(g)
    comm.deregister(b)
    comm.deregister(a)
    a.copy_(xs[rank])
    b.zero_()
    comm.all_reduce(a, b, "sum")  # staged again
    check(f"all_reduce after deregister {dtype}", b, want, tol)

st = comm.stats()
assert comm.status == 0 and st["timeouts"] == 0, (comm.status, st)
assert not fails, fails[:8]
print(f"RANK_OK {rank}", flush=True)
comm.close()
