#!/usr/bin/env python
"""Data-parallel ResNet-50 step throughput (images/s): bf16, 256 synthetic images per GPU,
SGD momentum 0.9, gradients in 25 MB buckets reduced by the fused all_reduce + 1/world scale
kernel on a communication stream while backward continues.

    torchrun --nproc-per-node N bench/dp_resnet50.py [--backend nvl|nccl] [--no-overlap]

`--backend nccl` runs the same harness over this library's NCCL wrapper; `--backend reference`
over the unmodified reference library (baseline/_ref, its NCCL backend: all_reduce then a separate
scale; the reference has no bf16, so 2-byte gradients are summed as float16).  Device-timed with
CUDA events, max over ranks, rank 0 prints one JSON line.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

import megray_b200 as mr  # noqa: E402
from megray_b200.models.resnet import resnet50, synthetic_batch  # noqa: E402
from megray_b200.parallel.data_parallel import GradBucketer  # noqa: E402


class ReferenceComm:
    """The few calls the harness needs, served by the reference library's public interface."""

    def __init__(self, world, rank, port):
        import ctypes as C

        path = os.path.join(ROOT, "baseline", "_ref", "libmegray_ref.so")
        if not os.path.exists(path):
            raise SystemExit("baseline/_ref/libmegray_ref.so is missing: run baseline/build_ref.py first")
        os.environ.setdefault("NCCL_LAUNCH_MODE", "PARALLEL")
        self._C = C
        self.ref = C.CDLL(path, mode=C.RTLD_LOCAL)
        self.ref.ref_comm_new.restype = C.c_void_p
        self.ref.ref_comm_init.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        self.ref.ref_all_reduce.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
        self.ref.ref_broadcast.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_uint, C.c_void_p]
        self.ref.ref_comm_delete.argtypes = [C.c_void_p]
        if rank == 0:
            assert self.ref.ref_create_server(world, port) == 0
        self.h = self.ref.ref_comm_new(world, rank)
        assert self.h and self.ref.ref_comm_init(self.h, b"127.0.0.1", port) == 0
        self.nranks, self.rank, self.backend = world, rank, -1

    def _stream(self):
        return self._C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def all_reduce(self, send, recv, op="sum"):
        code = {"sum": 0, "max": 1, "min": 2}[op]
        if send.dtype == torch.bfloat16:  # no bf16 in the reference: travel and add as float16
            tmp = send.to(torch.float16)
            assert self.ref.ref_all_reduce(self.h, tmp.data_ptr(), tmp.data_ptr(), tmp.numel(), 6, code, self._stream()) == 0
            recv.copy_(tmp)
            return
        dt = {torch.float32: 7, torch.float16: 6}[send.dtype]
        assert self.ref.ref_all_reduce(self.h, send.data_ptr(), recv.data_ptr(), send.numel(), dt, code, self._stream()) == 0

    def broadcast(self, send, recv, root):
        nbytes = recv.numel() * recv.element_size()
        assert self.ref.ref_broadcast(self.h, send.data_ptr(), recv.data_ptr(), nbytes, 1, root, self._stream()) == 0  # uint8

    def close(self):
        self.ref.ref_comm_delete(self.h)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="nvl")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--no-overlap", action="store_true")
    a = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    comm = server = None
    if world > 1:
        port = int(os.environ.get("MASTER_PORT", "29533")) + 3
        if a.backend == "reference":
            comm = ReferenceComm(world, rank, port)
        else:
            if rank == 0:
                server = mr.Server(world, port)
            comm = mr.Communicator(world, rank, a.backend).init("127.0.0.1", port)
    model = resnet50()
    bucketer = GradBucketer(model, comm, a.bucket_mb, overlap=not a.no_overlap)
    bucketer.broadcast_parameters(0)
    x, y = synthetic_batch(a.batch, seed=rank)
    loss_fn = torch.nn.CrossEntropyLoss()

    def step():
        bucketer.zero_grad()
        loss = loss_fn(model(x).float(), y)
        loss.backward()
        bucketer.sgd_step(lr=0.01, momentum=0.9)
        return loss

    for _ in range(a.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        loss = step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    if comm is not None:
        t = torch.tensor([ms], device="cuda")
        o = torch.empty_like(t)
        comm.all_reduce(t, o, "max")
        torch.cuda.synchronize()
        ms = float(o.item())
    if rank == 0:
        print(json.dumps({"metric": "DP ResNet-50 images/s", "value": a.batch * world / (ms / 1000.0),
                          "ms_per_step": ms, "n_gpus": world, "backend": a.backend if world > 1 else "none",
                          "batch_per_gpu": a.batch, "buckets_bytes": bucketer.bucket_bytes(),
                          "overlap": not a.no_overlap, "loss": float(loss.item())}), flush=True)
    if comm is not None:
        comm.close()


if __name__ == "__main__":
    main()
