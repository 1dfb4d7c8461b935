"""ResNet-50 for the data-parallel benchmark: torchvision's layout, random initialisation,
bf16 weights in channels-last memory format.  The convolutions are library (cuDNN) code; what
this library contributes to the benchmark is the gradient path (``parallel.data_parallel``)."""
from __future__ import annotations

import torch


def resnet50(device="cuda", dtype=torch.bfloat16, seed: int = 0) -> torch.nn.Module:
    import torchvision

    torch.manual_seed(seed)
    model = torchvision.models.resnet50(weights=None)  # ~25.6 M parameters, random init
    model = model.to(device=device, dtype=dtype)
    if str(device).startswith("cuda"):
        model = model.to(memory_format=torch.channels_last)
    return model


def synthetic_batch(batch: int, device="cuda", dtype=torch.bfloat16, seed: int = 0):
    """N(0,1) images of 3 x 224 x 224 and uniform labels over 1000 classes."""
    g = torch.Generator(device=device).manual_seed(seed)
    x = torch.randn(batch, 3, 224, 224, device=device, generator=g).to(dtype)
    if str(device).startswith("cuda"):
        x = x.contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 1000, (batch,), device=device, generator=g)
    return x, y
