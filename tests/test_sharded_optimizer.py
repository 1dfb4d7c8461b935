"""Sharded-state SGD (ZeRO stage 1) over the host backend: the weights follow exactly those of
momentum SGD on the mean gradient, while every rank holds 1/world of the momentum."""
import pytest
import torch

from helpers import with_group
from megray_b200.parallel.sharded_optimizer import ShardedSGD


def make_model():
    torch.manual_seed(5)
    return torch.nn.Sequential(torch.nn.Linear(7, 13), torch.nn.Tanh(), torch.nn.Linear(13, 5)).double()


def batch(rank, step):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randn(9, 7, generator=g, dtype=torch.float64), torch.randn(9, 5, generator=g, dtype=torch.float64)


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_matches_momentum_sgd_on_the_mean_gradient(n):
    steps, lr, mu, wd = 4, 0.05, 0.9, 0.01
    ref = make_model()
    opt = torch.optim.SGD(ref.parameters(), lr=lr, momentum=mu, weight_decay=wd)
    for s in range(steps):
        opt.zero_grad()
        loss = sum(((ref(x) - y) ** 2).mean() for x, y in (batch(r, s) for r in range(n))) / n
        loss.backward()
        opt.step()
    want = torch.cat([p.detach().reshape(-1) for p in ref.parameters()])

    models = [make_model() for _ in range(n)]  # built here: the global RNG is not thread-safe

    def body(comm, rank):
        model = models[rank]
        sh = ShardedSGD(model, comm if n > 1 else None, lr, mu, wd)
        sh.broadcast_parameters(0)
        for s in range(steps):
            sh.zero_grad()
            x, y = batch(rank, s)
            ((model(x) - y) ** 2).mean().backward()
            sh.step()
        total = sum(p.numel() for p in model.parameters())
        return sh.flat_w[:total].clone(), sh.state_bytes_per_rank(), total

    for flat, state_bytes, total in with_group(n, "shm", body):
        torch.testing.assert_close(flat, want, rtol=1e-9, atol=1e-11)
        assert state_bytes <= 8 * (total // n + 8)  # a 1/world share of the (float64 here) momentum
