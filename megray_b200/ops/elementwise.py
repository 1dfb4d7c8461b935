"""Memory-bound training kernels (src/kernels/elementwise.cu): fused SGD update and the
squared-error loss with its gradient."""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def sgd_step(w: torch.Tensor, g: torch.Tensor, lr: float, momentum_buf: torch.Tensor = None,
             momentum: float = 0.0, weight_decay: float = 0.0) -> None:
    """In place: w -= lr * (g + wd*w), or with an fp32 momentum buffer m = mu*m + g; w -= lr*m."""
    assert w.dtype == torch.bfloat16 and g.dtype == torch.bfloat16 and w.is_contiguous() and g.is_contiguous()
    mp = momentum_buf.data_ptr() if momentum_buf is not None else None
    rc = _lib.load().megray_sgd_bf16(w.data_ptr(), g.data_ptr(), mp, w.numel(), lr, momentum, weight_decay,
                                     _stream())
    if rc != 0:
        raise RuntimeError(f"megray_sgd_bf16 failed ({rc})")


def mse_loss_grad(y: torch.Tensor, target: torch.Tensor = None, scale: float = None,
                  dy: torch.Tensor = None):
    """Returns (loss, dy): loss = scale * sum((y - target)^2) as a 1-element fp32 tensor and
    dy = d loss / d y in bf16 (written into ``dy`` when given).  ``scale`` defaults to
    1 / y.numel() (mean)."""
    assert y.dtype == torch.bfloat16 and y.is_contiguous()
    if scale is None:
        scale = 1.0 / y.numel()
    loss = torch.zeros(1, dtype=torch.float32, device=y.device)
    if dy is None:
        dy = torch.empty_like(y)
    tp = target.data_ptr() if target is not None else None
    rc = _lib.load().megray_mse_bf16(y.data_ptr(), tp, dy.data_ptr(), loss.data_ptr(), y.numel(), scale,
                                     _stream())
    if rc != 0:
        raise RuntimeError(f"megray_mse_bf16 failed ({rc})")
    return loss, dy


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor = None, x_out: torch.Tensor = None,
                n_out: torch.Tensor = None, inv_rms: torch.Tensor = None, eps: float = 1e-6) -> None:
    """s = x + y (y optional); x_out = s; n_out = s * rsqrt(mean(s^2) + eps) per row; inv_rms = that
    factor (fp32, one per row).  Any of the outputs may be None."""
    rows, cols = x.shape
    assert x.dtype == torch.bfloat16 and x.is_contiguous()
    p = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    rc = _lib.load().megray_add_rmsnorm_bf16(p(x), p(y), p(x_out), p(n_out), p(inv_rms), rows, cols, eps,
                                             _stream())
    if rc != 0:
        raise RuntimeError(f"megray_add_rmsnorm_bf16 failed ({rc})")


def rmsnorm_bwd(dn: torch.Tensor, n: torch.Tensor, inv_rms: torch.Tensor, dres: torch.Tensor,
                dx: torch.Tensor) -> None:
    """dx = dres + inv_rms * (dn - n * mean(dn * n)) per row (dres optional)."""
    rows, cols = dn.shape
    p = lambda t: t.data_ptr() if t is not None else None  # noqa: E731
    rc = _lib.load().megray_rmsnorm_bwd_bf16(p(dn), p(n), p(inv_rms), p(dres), p(dx), rows, cols, _stream())
    if rc != 0:
        raise RuntimeError(f"megray_rmsnorm_bwd_bf16 failed ({rc})")
