"""Tensor-parallel MLP stack on n GPUs against the same model evaluated on one GPU: loss, output
shard and weight-gradient shards, for the fused (all_gather->GEMM, GEMM->reduce_scatter kernels)
and the unfused (collective then GEMM) paths."""
import torch
from common import setup

from megray_b200.models import TPMLPConfig, TPMLPStack
from megray_b200.ops import gemm_error_flag

rank, n, dev, comm, server = setup()
cfg = TPMLPConfig(d_model=512, ffn=1024, layers=2, tokens=max(1024, 256 * n), init_std=0.05, lr=0.0, seed=3)
g = torch.Generator(device=dev).manual_seed(11)
x_full = torch.randn(cfg.tokens, cfg.d_model, device=dev, generator=g).to(torch.bfloat16)
Ts = cfg.tokens // n

single = TPMLPStack(cfg, None, dev)
y_ref = single.forward(x_full).clone()
dy_full = (y_ref.float() * 1e-3).to(torch.bfloat16)
single.backward(dy_full)


def close(name, got, want, tol=3e-2):
    torch.cuda.synchronize()
    scale = max(float(want.float().abs().max()), 1e-6)
    err = float((got.float() - want.float()).abs().max()) / scale
    assert err < tol, f"{name}: relative error {err}"


for fused in (True, False):
    model = TPMLPStack(cfg, comm, dev, fused=fused)
    assert model.tp.fused == fused
    sl = slice(rank * Ts, (rank + 1) * Ts)
    y = model.forward(x_full[sl].contiguous())
    close(f"forward fused={fused}", y, y_ref[sl])
    dx = model.backward(dy_full[sl].contiguous())
    fl = cfg.ffn // n
    for l in range(cfg.layers):
        ref_gu = single.layers[l].g_gu
        want_gu = torch.cat([ref_gu[rank * fl:(rank + 1) * fl], ref_gu[cfg.ffn + rank * fl: cfg.ffn + (rank + 1) * fl]])
        close(f"g_gu[{l}] fused={fused}", model.layers[l].g_gu, want_gu)
        close(f"g_down[{l}] fused={fused}", model.layers[l].g_down, single.layers[l].g_down[:, rank * fl:(rank + 1) * fl])
    # a second forward re-uses every buffer and flag block
    y2 = model.forward(x_full[sl].contiguous())
    close(f"forward again fused={fused}", y2, y_ref[sl])
    assert int(gemm_error_flag(dev).item()) == 0 and comm.status == 0

print(f"RANK_OK {rank}", flush=True)
comm.close()
