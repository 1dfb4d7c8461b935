"""Shared set-up of the multi-GPU test scripts (one process per GPU under torchrun)."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import megray_b200 as mr  # noqa: E402


def setup(backend="nvl", port_offset=1):
    rank = int(os.environ["RANK"])
    n = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    port = int(os.environ.get("MASTER_PORT", "29641")) + port_offset
    server = mr.Server(n, port) if rank == 0 else None
    comm = mr.Communicator(n, rank, backend).init("127.0.0.1", port)
    return rank, n, torch.device("cuda", local), comm, server
