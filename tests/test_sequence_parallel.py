"""Ulysses head / sequence swap and ring attention over the host backend (CPU tensors, ranks as
threads): the sharded computations reproduce attention over the whole sequence."""
import math

import pytest
import torch

from helpers import with_group
from megray_b200.parallel.sequence_parallel import heads_to_seq, ring_attention, seq_to_heads, ulysses_attention


def full_attention(q, k, v, causal):
    scores = torch.einsum("qhd,khd->hqk", q.double(), k.double()) / math.sqrt(q.shape[-1])
    if causal:
        s = q.shape[0]
        mask = torch.triu(torch.ones(s, s, dtype=torch.bool), diagonal=1)
        scores = scores.masked_fill(mask[None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), v.double())


def make(S, H, D, seed):
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(S, H, D, generator=g) for _ in range(3))


@pytest.mark.parametrize("n", [1, 2, 4])
def test_head_sequence_swap_round_trip(n):
    S, H, D = 8 * n, 4 * n, 3
    x = torch.arange(S * H * D, dtype=torch.float32).reshape(S, H, D)

    def body(comm, rank):
        mine = x[rank * S // n:(rank + 1) * S // n].contiguous()
        heads = seq_to_heads(comm, mine)
        back = heads_to_seq(comm, heads)
        return heads, back

    for rank, (heads, back) in enumerate(with_group(n, "shm", body)):
        hl = H // n
        assert torch.equal(heads, x[:, rank * hl:(rank + 1) * hl])
        assert torch.equal(back, x[rank * S // n:(rank + 1) * S // n])


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_ulysses_attention_matches_full_attention(n, causal):
    S, H, D = 16 * n, 2 * n, 8
    q, k, v = make(S, H, D, 1)
    want = full_attention(q, k, v, causal)

    def body(comm, rank):
        sl = slice(rank * S // n, (rank + 1) * S // n)
        return ulysses_attention(comm, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), causal)

    for rank, out in enumerate(with_group(n, "shm", body)):
        torch.testing.assert_close(out.double(), want[rank * S // n:(rank + 1) * S // n], rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n", [1, 2, 3, 4])
@pytest.mark.parametrize("causal", [False, True])
def test_ring_attention_matches_full_attention(n, causal):
    S, H, D = 12 * n, 3, 8
    q, k, v = make(S, H, D, 2)
    want = full_attention(q, k, v, causal)

    def body(comm, rank):
        sl = slice(rank * S // n, (rank + 1) * S // n)
        return ring_attention(comm, q[sl].contiguous(), k[sl].contiguous(), v[sl].contiguous(), causal)

    for rank, out in enumerate(with_group(n, "shm", body)):
        torch.testing.assert_close(out.double(), want[rank * S // n:(rank + 1) * S // n], rtol=1e-5, atol=1e-5)


def test_heads_must_divide():
    def body(comm, rank):
        with pytest.raises(ValueError):
            seq_to_heads(comm, torch.zeros(4, 3, 2))
        return True

    assert all(with_group(2, "shm", body))
