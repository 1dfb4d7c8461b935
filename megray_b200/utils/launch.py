"""Process-per-GPU start-up (torchrun style environment) for the harnesses."""
from __future__ import annotations

import os

from .. import comm as _comm


def init_from_env(backend: str = "nvl", port_offset: int = 1):
    """Reads RANK / LOCAL_RANK / WORLD_SIZE / MASTER_PORT, selects this rank's GPU, starts the
    rendezvous server on rank 0 (127.0.0.1, MASTER_PORT + port_offset) and returns
    ``(rank, world, device, communicator or None, server or None)``.  With one rank no
    communicator is created."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world == 1:
        return rank, world, device, None, None
    port = int(os.environ.get("MASTER_PORT", "29533")) + port_offset
    server = _comm.Server(world, port) if rank == 0 else None
    communicator = _comm.Communicator(world, rank, backend).init("127.0.0.1", port)
    return rank, world, device, communicator, server


def max_over_ranks(communicator, value: float, device=None) -> float:
    """The largest ``value`` over all ranks (device-side all_reduce MAX); identity for one rank."""
    if communicator is None:
        return value
    import torch

    t = torch.tensor([value], device=device or "cuda", dtype=torch.float32)
    o = torch.empty_like(t)
    communicator.all_reduce(t, o, "max")
    torch.cuda.synchronize()
    return float(o.item())
