"""Ranks in separate processes on ordinary torch tensors: allocations are exported and mapped on
first use and the single-pass kernels run on them (run under torchrun)."""
import torch
from common import setup

rank, n, dev, comm, server = setup()
fails = []


def expect(name, got, want):
    torch.cuda.synchronize()
    if not torch.equal(got.cpu(), want):
        fails.append(name)


numel = (1 << 20) + 8  # 4 MiB of float32: far above the small-message limit
want_sum = torch.full((numel,), float(sum(range(1, n + 1))))

# 1. a rank that keeps bringing new allocations while its peers reuse theirs: only that rank exports,
#    and the peers' kernels wait for their helper threads to map what it exported
keep = torch.full((numel,), rank + 1.0, device=dev)
out = torch.empty_like(keep)
held = []
for it in range(4):
    if rank == 0:
        x = torch.full((numel + 4096 * it,), rank + 1.0, device=dev)[:numel]  # another allocation every time
        held.append(x)
    else:
        x = keep
    comm.all_reduce(x, out)
    expect(f"all_reduce, new allocation on rank 0, round {it}", out, want_sum)

# 2. memory that was freed and allocated again at (most likely) the same address gets a new entry
big = torch.full((8 * numel,), rank + 1.0, device=dev)
comm.all_reduce(big[:numel], out)
expect("all_reduce before free", out, want_sum)
torch.cuda.synchronize()
comm.stream_barrier()
torch.cuda.synchronize()
addr = big.data_ptr()
del big
torch.cuda.empty_cache()
big = torch.full((8 * numel,), 2.0 * (rank + 1), device=dev)
comm.all_reduce(big[:numel], out)
expect(f"all_reduce after free (same address: {big.data_ptr() == addr})", out, 2 * want_sum)

# 3. every operation once, on views at odd offsets inside one allocation
pool = torch.arange(4 * numel * n + 64, dtype=torch.float32, device=dev) + 1000.0 * rank
m = numel // 2
src = pool[3:3 + m * n]
root = n - 1
host = [torch.arange(4 * numel * n + 64, dtype=torch.float32) + 1000.0 * q for q in range(n)]
o = torch.empty(m * n, dtype=torch.float32, device=dev)
comm.all_gather(src[:m], o)
expect("all_gather", o, torch.cat([host[q][3:3 + m] for q in range(n)]))
comm.all_to_all(src, o)
expect("all_to_all", o, torch.cat([host[q][3 + rank * m:3 + (rank + 1) * m] for q in range(n)]))
o1 = torch.empty(m, dtype=torch.float32, device=dev)
comm.reduce_scatter(src, o1, "max")
expect("reduce_scatter max", o1, host[n - 1][3 + rank * m:3 + (rank + 1) * m])
comm.broadcast(src[:m], o1, root)
expect("broadcast", o1, host[root][3:3 + m])
comm.scatter(src if rank == root else None, o1, root)
expect("scatter", o1, host[root][3 + rank * m:3 + (rank + 1) * m])
o2 = torch.zeros(m, dtype=torch.float32, device=dev)
comm.reduce(src[:m], o2, root, "min")
if rank == root:
    expect("reduce min", o2, host[0][3:3 + m])
big_out = torch.empty(m * n, dtype=torch.float32, device=dev) if rank == root else None
comm.gather(src[:m], big_out, root)
if rank == root:
    expect("gather", big_out, torch.cat([host[q][3:3 + m] for q in range(n)]))
# a reduce large enough for the form in which the root pushes its input
wide = torch.full((6 * numel,), rank + 1.0, device=dev)
wide_out = torch.zeros(6 * numel, device=dev) if rank == 0 else None
comm.reduce(wide, wide_out, 0, "sum")
if rank == 0:
    expect("reduce 24 MiB", wide_out, torch.full((6 * numel,), float(sum(range(1, n + 1)))))

# 4. a call larger than what is exported automatically: staged until the buffers are registered
huge = torch.full((20 * numel,), rank + 1.0, device=dev)  # 80 MiB
huge_out = torch.empty_like(huge)
before = comm.stats()["direct"]
comm.all_reduce(huge, huge_out)
expect("all_reduce 80 MiB, not registered", huge_out, torch.full((20 * numel,), float(sum(range(1, n + 1)))))
assert comm.stats()["direct"] == before, "a large call on memory no peer has mapped must not wait for mappings in a kernel"
assert comm.register(huge) and comm.register(huge_out)
comm.all_reduce(huge, huge_out)
expect("all_reduce 80 MiB, registered", huge_out, torch.full((20 * numel,), float(sum(range(1, n + 1)))))
assert comm.stats()["direct"] == before + 1, comm.stats()

st = comm.stats()
assert st["timeouts"] == 0 and comm.status == 0, (st, comm.status)
assert st["direct"] >= 10, st  # the single-pass kernels ran, not the staged ones
assert not fails, fails[:10]
print(f"RANK_OK {rank} direct={st['direct']}", flush=True)
comm.close()
