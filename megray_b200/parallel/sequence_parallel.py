"""Long-sequence parallelism on top of the communicator: the Ulysses head / sequence swap and
ring attention.

Both work on torch tensors of any device the communicator's backend serves (CUDA tensors on the
NVL or NCCL backend, CPU tensors on the host backend, which is how the tests run without a GPU).

* Ulysses: activations are sharded on the sequence, ``[S/n, H, D]`` per rank.  One all_to_all
  turns them into ``[S, H/n, D]`` (all positions, a slice of the heads), attention runs locally
  on whole sequences, and a second all_to_all swaps back.  The all_to_all moves equal chunks, the
  form the reference library offers (include/megray/communicator.h:75-77); the re-layout around
  it is done here.
* Ring attention (context parallelism): queries stay put, key / value blocks travel around the
  ring of ranks with grouped send / recv (include/megray/communicator.h:51-57,107-109 in the
  reference: the primitives; no attention code exists there) while a running soft-max
  (maximum, denominator, weighted sum in fp32) absorbs one block per step.  With ``causal=True``
  blocks that lie entirely in the future are skipped and the diagonal block is masked.

The attention arithmetic itself is plain torch; what this module contributes is the
communication schedule.
"""
from __future__ import annotations

import math

import torch


# ---------------------------------------------------------------------------------- Ulysses
def seq_to_heads(comm, x: torch.Tensor) -> torch.Tensor:
    """``[S/n, H, D]`` (this rank's positions, all heads) -> ``[S, H/n, D]`` (all positions, this
    rank's heads).  H must be divisible by the number of ranks."""
    n = comm.nranks
    s_loc, heads, dim = x.shape
    if heads % n:
        raise ValueError("the number of heads must be divisible by the number of ranks")
    if n == 1:
        return x.contiguous()
    hl = heads // n
    # chunk q of the send buffer: my positions of rank q's heads
    send = x.reshape(s_loc, n, hl, dim).permute(1, 0, 2, 3).contiguous()
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv)
    # chunk q of the receive buffer: rank q's positions of my heads, ranks in sequence order
    return recv.reshape(n * s_loc, hl, dim)


def heads_to_seq(comm, y: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`seq_to_heads`: ``[S, H/n, D]`` -> ``[S/n, H, D]``."""
    n = comm.nranks
    s_all, hl, dim = y.shape
    if s_all % n:
        raise ValueError("the sequence length must be divisible by the number of ranks")
    if n == 1:
        return y.contiguous()
    s_loc = s_all // n
    send = y.reshape(n, s_loc, hl, dim).contiguous()  # chunk q: rank q's positions of my heads
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv)
    # chunk q: my positions of rank q's heads -> heads in rank order
    return recv.permute(1, 0, 2, 3).reshape(s_loc, n * hl, dim)


def ulysses_attention(comm, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """Attention over the whole sequence for sequence-sharded ``[S/n, H, D]`` inputs: swap to head
    shards, attend locally, swap back."""
    qh, kh, vh = (seq_to_heads(comm, t) for t in (q, k, v))
    out = _attention(qh, kh, vh, causal, 0, 0)
    return heads_to_seq(comm, out.to(q.dtype))


# ---------------------------------------------------------------------------------- ring attention
def _attention(q, k, v, causal, q_start, k_start):
    """softmax(q k^T / sqrt(D)) v for [Sq, H, D] x [Sk, H, D] in fp32; positions start at
    ``q_start`` / ``k_start`` for the causal mask."""
    qf, kf, vf = q.float(), k.float(), v.float()
    scores = torch.einsum("qhd,khd->hqk", qf, kf) / math.sqrt(q.shape[-1])
    if causal:
        qi = torch.arange(q.shape[0], device=q.device) + q_start
        ki = torch.arange(k.shape[0], device=k.device) + k_start
        scores = scores.masked_fill(ki[None, None, :] > qi[None, :, None], float("-inf"))
    return torch.einsum("hqk,khd->qhd", torch.softmax(scores, dim=-1), vf)


def ring_attention(comm, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = False) -> torch.Tensor:
    """Attention over the whole sequence for sequence-sharded ``[S/n, H, D]`` inputs (rank r holds
    positions ``[r S/n, (r+1) S/n)``).  Key / value blocks go around the ring; every step folds
    one block into the running soft-max.  Returns ``[S/n, H, D]`` in the dtype of ``q``."""
    n, r = comm.nranks, comm.rank
    s_loc, heads, dim = q.shape
    scale = 1.0 / math.sqrt(dim)
    qf = q.float()
    m = torch.full((heads, s_loc), float("-inf"), device=q.device)       # running maximum
    l = torch.zeros(heads, s_loc, device=q.device)                        # running denominator
    acc = torch.zeros(s_loc, heads, dim, device=q.device)                 # running weighted sum
    kv = torch.stack([k, v]).contiguous()                                 # travels as one message
    nxt, prv = (r + 1) % n, (r - 1) % n
    for step in range(n):
        src = (r - step) % n  # the rank whose block is here now
        if step + 1 < n:
            # pass the block on (stream-ordered on the CUDA backends, so it overlaps this step's
            # arithmetic; the receive lands in a second buffer)
            incoming = torch.empty_like(kv)
            comm.group_start()
            comm.send(kv, nxt)
            comm.recv(incoming, prv)
            comm.group_end()
        if not (causal and src > r):  # a block entirely in the future contributes nothing
            kb, vb = kv[0].float(), kv[1].float()
            scores = torch.einsum("qhd,khd->hqk", qf, kb) * scale
            if causal and src == r:
                idx = torch.arange(s_loc, device=q.device)
                scores = scores.masked_fill(idx[None, None, :] > idx[None, :, None], float("-inf"))
            m_new = torch.maximum(m, scores.amax(dim=-1))
            p = torch.exp(scores - m_new[..., None])
            corr = torch.exp(m - m_new)
            l = l * corr + p.sum(dim=-1)
            acc = acc * corr.transpose(0, 1)[..., None] + torch.einsum("hqk,khd->qhd", p, vb)
            m = m_new
        if step + 1 < n:
            kv = incoming
    return (acc / l.transpose(0, 1)[..., None]).to(q.dtype)
