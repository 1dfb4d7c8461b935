#!/usr/bin/env python
"""Data-parallel ResNet-50 step throughput (images/s): bf16, 256 synthetic images per GPU,
SGD momentum 0.9, gradients in 25 MB buckets reduced by the fused all_reduce + 1/world scale
kernel on a communication stream while backward continues.

    torchrun --nproc-per-node N bench/dp_resnet50.py [--backend nvl|nccl] [--no-overlap]

`--backend nccl` runs the same harness over the NCCL wrapper (the baseline path).  Device-timed
with CUDA events, max over ranks, rank 0 prints one JSON line.
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
