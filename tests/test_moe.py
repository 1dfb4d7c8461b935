"""MoE layer on one GPU (all experts local) against a float32 PyTorch evaluation: routing,
output, input gradient, gate gradient and expert weight gradients."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def reference(x, logits, w_gu, w_down, E, F, H):
    top = logits.topk(2, dim=1)
    idx = top.indices
    w = torch.softmax(top.values, dim=1)
    out = torch.zeros(x.shape[0], H, device=x.device)
    for e in range(E):
        wg = w_gu[e * 2 * F:(e + 1) * 2 * F]
        wd = w_down[e * H:(e + 1) * H]
        for k in range(2):
            sel = (idx[:, k] == e).nonzero().flatten()
            if sel.numel() == 0:
                continue
            gu = x[sel] @ wg.t()
            h = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
            out.index_add_(0, sel, (h @ wd.t()) * w[sel, k:k + 1])
    return out, idx, w


def test_moe_layer_matches_float32_model():
    from megray_b200.models import MoEConfig, MoELayer
    from megray_b200.ops import gemm_error_flag

    torch.manual_seed(0)
    cfg = MoEConfig(experts=8, hidden=256, ffn=384, tokens=1000, init_std=0.05, lr=0.0, capacity_factor=2.0)
    layer = MoELayer(cfg)
    x = torch.randn(cfg.tokens, cfg.hidden, device="cuda").to(torch.bfloat16)
    logits = torch.randn(cfg.tokens, cfg.experts, device="cuda")
    y = layer.forward(x, logits)
    torch.cuda.synchronize()
    assert not layer.ep.overflowed()

    xf = x.float().requires_grad_()
    lf = logits.clone().requires_grad_()
    wgu = layer.w_gu.float().requires_grad_()
    wdn = layer.w_down.float().requires_grad_()
    want, idx, w = reference(xf, lf, wgu, wdn, cfg.experts, cfg.ffn, cfg.hidden)
    assert torch.equal(layer.ep.idx.long(), idx)
    assert torch.allclose(layer.ep.w, w, atol=1e-5)
    # every (token, slot) landed on a distinct row inside its expert's segment
    pos = layer.ep.pos.flatten().cpu()
    assert pos.unique().numel() == pos.numel()
    scale = float(want.abs().max())
    assert float((y.float() - want).abs().max()) < 3e-2 * scale

    dout = (torch.randn_like(want) * 0.1).to(torch.bfloat16)
    dx, dlogits = layer.backward(dout)
    want.backward(dout.float())
    torch.cuda.synchronize()
    assert int(gemm_error_flag().item()) == 0

    def close(got, ref, tol=4e-2):
        s = max(float(ref.abs().max()), 1e-6)
        assert float((got.float() - ref).abs().max()) < tol * s

    close(dx, xf.grad)
    close(dlogits, lf.grad)
    close(layer.g_gu, wgu.grad)
    close(layer.g_down, wdn.grad)


def test_plan_flags_an_overflowing_owner():
    from megray_b200.models import MoEConfig, MoELayer

    cfg = MoEConfig(experts=4, hidden=256, ffn=128, tokens=512, capacity_factor=0.25)
    layer = MoELayer(cfg)
    logits = torch.zeros(cfg.tokens, cfg.experts, device="cuda")
    layer.ep.route(logits)
    layer.ep.plan()
    assert layer.ep.overflowed()
