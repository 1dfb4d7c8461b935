"""Operators backed by the library's own sm_100a kernels."""
from .gemm import (EPI_ACCUM, EPI_DSWIGLU, EPI_PUSH, EPI_STORE, EPI_STORE_F32, EPI_STORE_ROWS, EPI_SWIGLU, build_gemm_args, gemm, gemm_split_k, pick_split_k,
                   gemm_error_flag)  # noqa: F401
from .elementwise import add_rmsnorm, mse_loss_grad, rmsnorm_bwd, sgd_step  # noqa: F401
