"""Expert-parallel MoE layer over n GPUs against the same layer with all experts on one GPU
(evaluated on this rank's tokens): outputs, input gradients, gate gradients, and expert weight
gradients (which sum the contributions of every rank's tokens)."""
import torch
from common import setup

from megray_b200.models import MoEConfig, MoELayer
from megray_b200.ops import gemm_error_flag

rank, n, dev, comm, server = setup()
cfg = MoEConfig(experts=8, hidden=256, ffn=384, tokens=768, init_std=0.05, lr=0.0, capacity_factor=2.0, seed=5)
g = torch.Generator(device=dev).manual_seed(100 + rank)
x = torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g).to(torch.bfloat16)
logits = torch.randn(cfg.tokens, cfg.experts, device=dev, generator=g)
dout = (torch.randn(cfg.tokens, cfg.hidden, device=dev, generator=g) * 0.1).to(torch.bfloat16)

local = MoELayer(cfg, None, dev)        # all 8 experts here
y_ref = local.forward(x, logits).clone()
dx_ref, dl_ref = local.backward(dout)
dx_ref, dl_ref = dx_ref.clone(), dl_ref.clone()

ep = MoELayer(cfg, comm, dev)           # 8 / n experts here


def close(name, got, want, tol=4e-2):
    torch.cuda.synchronize()
    s = max(float(want.float().abs().max()), 1e-6)
    err = float((got.float() - want.float()).abs().max()) / s
    assert err < tol, f"{name}: {err}"


for it in range(2):  # the second pass re-uses every buffer
    y = ep.forward(x, logits)
    close("forward", y, y_ref)
    dx, dl = ep.backward(dout)
    close("dx", dx, dx_ref)
    close("dlogits", dl, dl_ref)
    # weight gradients: sum of all ranks' single-GPU gradients, then this rank's experts
    El, F, H = cfg.experts // n, cfg.ffn, cfg.hidden
    for name, mine, ref, rows in (("g_gu", ep.g_gu, local.g_gu, 2 * F), ("g_down", ep.g_down, local.g_down, H)):
        tot = torch.empty_like(ref, dtype=torch.float32)
        comm.all_reduce(ref.float().contiguous(), tot)
        close(name, mine, tot[rank * El * rows:(rank + 1) * El * rows])
    assert not ep.ep.overflowed()
assert int(gemm_error_flag(dev).item()) == 0 and comm.status == 0
print(f"RANK_OK {rank}", flush=True)
comm.close()
