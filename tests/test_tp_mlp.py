"""The flagship model on one GPU: one training step against a float32 PyTorch evaluation, and
the memory-bound training kernels (SGD update, squared-error loss)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_smoke_entry_point():
    import __graft_entry__ as entry

    entry.smoke()


def test_sgd_and_loss_kernels():
    from megray_b200.ops import mse_loss_grad, sgd_step

    torch.manual_seed(0)
    w = torch.randn(100_003, device="cuda").to(torch.bfloat16)
    g = torch.randn_like(w)
    w0 = w.float().clone()
    sgd_step(w, g, 0.1)
    want = w0 - 0.1 * g.float()
    # fused multiply-add in the kernel against separate roundings: within one bf16 step
    assert torch.allclose(w.float(), want, rtol=2 ** -7, atol=1e-6)
    m = torch.zeros(w.numel(), device="cuda")
    w2 = w.clone()
    sgd_step(w2, g, 0.1, momentum_buf=m, momentum=0.9)
    assert torch.allclose(m, g.float())
    assert torch.allclose(w2.float(), w.float() - 0.1 * g.float(), rtol=2 ** -7, atol=1e-6)
    y = torch.randn(333, 77, device="cuda").to(torch.bfloat16)
    loss, dy = mse_loss_grad(y)
    assert abs(float(loss.item()) - float(y.float().pow(2).mean())) < 1e-4
    assert torch.allclose(dy.float(), (2 * y.float() / y.numel()).to(torch.bfloat16).float())


def test_two_steps_reduce_the_loss():
    from megray_b200.models import TPMLPConfig, TPMLPStack

    cfg = TPMLPConfig(d_model=256, ffn=512, layers=2, tokens=256, init_std=0.05, lr=5e-2)
    model = TPMLPStack(cfg)
    x = torch.randn(cfg.tokens, cfg.d_model, device="cuda").to(torch.bfloat16)
    first = float(model.train_step_device(x).item())
    for _ in range(3):
        last = float(model.train_step_device(x).item())
    assert last < first


def test_add_rmsnorm_forward_and_backward():
    from megray_b200.ops import add_rmsnorm, rmsnorm_bwd

    torch.manual_seed(1)
    rows, cols = 37, 1024
    x = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    y = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    s_out, n_out = torch.empty_like(x), torch.empty_like(x)
    inv = torch.empty(rows, device="cuda")
    add_rmsnorm(x, y, s_out, n_out, inv)
    s = (x.float() + y.float()).to(torch.bfloat16)
    assert torch.equal(s_out, s)
    sf = s.float().requires_grad_()
    want = torch.nn.functional.rms_norm(sf, (cols,), eps=1e-6)
    assert torch.allclose(n_out.float(), want, rtol=1e-2, atol=1e-2)
    dn = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    dres = torch.randn(rows, cols, device="cuda").to(torch.bfloat16)
    dx = torch.empty_like(x)
    rmsnorm_bwd(dn, n_out, inv, dres, dx)
    want.backward(dn.float())
    assert torch.allclose(dx.float(), sf.grad + dres.float(), rtol=2e-2, atol=2e-2)
