"""Gradient bucketing on CPU ranks (host backend): the averaged gradients of two data-parallel
ranks equal the gradient of the full batch on one model, buckets split at the size limit, and a
step through the bucketed SGD keeps the ranks' weights identical."""
import numpy as np
import torch

from helpers import with_group
from megray_b200.parallel.data_parallel import GradBucketer


def make_model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 32), torch.nn.Tanh(),
                               torch.nn.Linear(32, 4))


def test_bucketed_average_equals_full_batch_gradient():
    torch.manual_seed(1)
    x = torch.randn(8, 16)
    y = torch.randn(8, 4)
    ref = make_model()
    torch.nn.functional.mse_loss(ref(x), y).backward()
    want = [p.grad.clone() for p in ref.parameters()]

    # built on the main thread: the global RNG is shared by the rank threads
    models = [make_model(seed=0), make_model(seed=7)]  # rank 1 starts different: broadcast fixes it

    def body(comm, rank):
        model = models[rank]
        b = GradBucketer(model, comm, bucket_mb=0.003, overlap=False)  # ~3 KB: several buckets
        b.broadcast_parameters(0)
        xs, ys = x[rank * 4:(rank + 1) * 4], y[rank * 4:(rank + 1) * 4]
        b.zero_grad()
        torch.nn.functional.mse_loss(model(xs), ys).backward()
        b.wait()
        grads = [p.grad.clone() for p in model.parameters()]
        b.sgd_step(lr=0.1, momentum=0.9)
        return grads, [p.detach().clone() for p in model.parameters()], b.bucket_bytes()

    res = with_group(2, "shm", body)
    for grads, _, sizes in res:
        assert len(sizes) > 1 and all(s <= 3200 or len(sizes) > 1 for s in sizes)
        for g, w in zip(grads, want):
            np.testing.assert_allclose(g.numpy(), w.numpy(), rtol=1e-5, atol=1e-6)
    for a, b in zip(res[0][1], res[1][1]):
        assert torch.equal(a, b)  # identical weights after the step
