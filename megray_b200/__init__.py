"""megray_b200: a B200-native collective communication library with MegRay's interface.

Native code lives in ``libmegray.so`` (built in-tree by ``python -m megray_b200.build``);
this package is its PyTorch-facing layer: communicators over tensors (``comm``), the
tcgen05 GEMM and fused operators (``ops``), parallelism harnesses (``parallel``) and
the model families used by the benchmarks (``models``).
"""
from .comm import (  # noqa: F401
    BACKENDS, BFLOAT16, CHAR, FLOAT16, FLOAT32, FLOAT64, INT8, INT32, INT64, MAX, MIN, NCCL, NVL,
    RCCL, SHM, SUM, UCX, UINT8, UINT32, UINT64, Client, Communicator, MegRayError, Server,
    create_server, get_communicator, get_free_port, get_host_ip,
)

__version__ = "0.1.0"
