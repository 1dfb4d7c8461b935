"""The benchmark's full-size tensor-parallel step (d_model 8192, ffn 28672, 32768 tokens, two
layers) through the fused kernels and through collective-then-GEMM, on the same weights and
tokens: output shard, input-gradient shard and every weight-gradient shard are compared element
by element.  Both paths round each rank's partial products to bf16 and add them in rank order in
float32, so they must agree to the last bit or nearly (a tolerance of one bf16 step is allowed)."""
import os

import torch
from common import setup

from megray_b200.models import TPMLPConfig, TPMLPStack
from megray_b200.ops import gemm_error_flag

os.environ.setdefault("MEGRAY_HEAP_MB", "6144")
rank, n, dev, comm, server = setup()
cfg = TPMLPConfig(d_model=8192, ffn=28672, layers=2, tokens=32768, lr=0.0)
g = torch.Generator(device=dev).manual_seed(1234 + rank)
x = torch.randn(cfg.tokens // n, cfg.d_model, device=dev, generator=g).to(torch.bfloat16)

results = {}
for fused in (True, False):
    model = TPMLPStack(cfg, comm, dev, fused=fused)
    assert model.tp.fused == fused
    y = model.forward(x).clone()
    dy = (y.float() * 1e-3).to(torch.bfloat16)
    dx = model.backward(dy).clone()
    torch.cuda.synchronize()
    flag, status = int(gemm_error_flag(dev).item()), comm.status
    assert flag == 0 and status == 0, f"fused={fused}: GEMM error flag {flag}, communicator status {status}"
    results[fused] = (y, dx, [l.g_gu.clone() for l in model.layers], [l.g_down.clone() for l in model.layers])
    del model
    torch.cuda.empty_cache()


def compare(name, a, b):
    a, b = a.float(), b.float()
    scale = max(float(b.abs().max()), 1e-9)
    worst = float((a - b).abs().max()) / scale
    differ = int((a != b).sum())
    assert worst <= 2 ** -7, f"{name}: fused and unfused differ by {worst} of the largest value"
    return f"{name}: {differ}/{a.numel()} elements differ, worst {worst:.2e}"


fy, fdx, fgu, fgd = results[True]
uy, udx, ugu, ugd = results[False]
lines = [compare("output shard", fy, uy), compare("input-gradient shard", fdx, udx)]
for l in range(cfg.layers):
    lines.append(compare(f"g_gu[{l}]", fgu[l], ugu[l]))
    lines.append(compare(f"g_down[{l}]", fgd[l], ugd[l]))
if rank == 0:
    print("\n".join(lines), flush=True)
print(f"RANK_OK {rank}", flush=True)
comm.close()
