"""1F1B pipeline over the host backend (CPU tensors, one thread per stage): outputs, input
gradients and weight gradients equal those of the same layers run in one process."""
import pytest
import torch

from helpers import with_group
from megray_b200.parallel.pipeline import PipelineStage, one_f_one_b


@pytest.mark.parametrize("P,M", [(1, 3), (2, 1), (2, 4), (3, 2), (4, 8), (4, 3)])
def test_schedule_shape(P, M):
    for s in range(P):
        order = one_f_one_b(P, M, s)
        assert [m for k, m in order if k == "F"] == list(range(M))
        assert [m for k, m in order if k == "B"] == list(range(M))
        alive = peak = 0
        for k, m in order:
            assert k == "F" or ("F", m) in order[: order.index((k, m))]  # backward after its forward
            alive += 1 if k == "F" else -1
            peak = max(peak, alive)
        assert peak <= min(P - s, M)  # at most P - s micro-batches in flight on stage s


@pytest.mark.parametrize("P,M", [(2, 1), (2, 5), (3, 4), (4, 8), (4, 2)])
def test_1f1b_matches_single_process_autograd(P, M):
    torch.manual_seed(0)
    B, D = 6, 16
    weights = [torch.randn(D, D, dtype=torch.float64) * 0.3 for _ in range(P)]
    xs = [torch.randn(B, D, dtype=torch.float64) for _ in range(M)]
    targets = [torch.randn(B, D, dtype=torch.float64) for _ in range(M)]

    # one process: all layers, all micro-batches, gradients accumulate
    ws = [w.clone().requires_grad_() for w in weights]
    xr = [x.clone().requires_grad_() for x in xs]
    outs_ref = []
    for mb in range(M):
        h = xr[mb]
        for w in ws:
            h = torch.tanh(h @ w)
        outs_ref.append(h.detach())
        ((h - targets[mb]) ** 2).sum().backward()

    def body(comm, rank):
        w = weights[rank].clone().requires_grad_()
        saved = {}

        def forward(mb, x):
            x = x.clone().requires_grad_()
            y = torch.tanh(x @ w)
            saved[mb] = (x, y)
            return y.detach()

        def backward(mb, dy):
            x, y = saved.pop(mb)
            y.backward(dy)
            return x.grad

        stage = PipelineStage(comm, forward, backward, (B, D), dtype=torch.float64)
        dxs = {}
        if rank == 0:  # keep the input gradients of the first stage for the comparison
            inner = stage.backward

            def keep(mb, dy):
                dxs[mb] = inner(mb, dy)
                return dxs[mb]

            stage.backward = keep
        outs = stage.run(M, inputs=xs if rank == 0 else None,
                         loss_grad=(lambda mb, y: 2 * (y - targets[mb])) if rank == P - 1 else None)
        assert not saved
        return w.grad, outs, dxs

    res = with_group(P, "shm", body)
    for s, (gw, outs, dxs) in enumerate(res):
        torch.testing.assert_close(gw, ws[s].grad, rtol=1e-10, atol=1e-10)
    for mb in range(M):
        torch.testing.assert_close(res[P - 1][1][mb], outs_ref[mb], rtol=1e-10, atol=1e-10)
        torch.testing.assert_close(res[0][2][mb], xr[mb].grad, rtol=1e-10, atol=1e-10)
