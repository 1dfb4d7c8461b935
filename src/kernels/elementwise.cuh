// Small memory-bound kernels used by the training harnesses: fused SGD update,
// squared-error loss with its gradient, casts and fills.  The reference has no
// such kernels (it is a pure communication library).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgk {
namespace ew {

// w -= lr * (g + wd * w), optionally with momentum: m = mu*m + g'; w -= lr*m.
// bf16 weights and gradients, fp32 arithmetic; `momentum` buffer is fp32 or null.
cudaError_t launch_sgd_bf16(void* w, const void* g, float* momentum, uint64_t n, float lr, float mu,
                            float weight_decay, cudaStream_t stream);

// loss_out[0] += sum((y - target)^2) * scale; dy = 2 * (y - target) * scale (bf16), target may
// be null (zero target).  `loss_out` must be zeroed by the caller.
cudaError_t launch_mse_bf16(const void* y, const void* target, void* dy, float* loss_out, uint64_t n,
                            float scale, cudaStream_t stream);

// Fused residual add + RMS normalisation over rows of `cols` bf16 elements (cols % 8 == 0,
// cols <= 16384):  s = x + y (y may be null);  x_out = s (if non-null);
// n_out = s * rsqrt(mean(s^2) + eps) (if non-null);  inv_rms[row] = that factor (if non-null).
cudaError_t launch_add_rmsnorm_bf16(const void* x, const void* y, void* x_out, void* n_out,
                                    float* inv_rms, int rows, int cols, float eps,
                                    cudaStream_t stream);

// Backward of n = s * inv_rms with the residual gradient added:
//   dx = dres + inv_rms * (dn - n * mean(dn * n))      (dres may be null)
cudaError_t launch_rmsnorm_bwd_bf16(const void* dn, const void* n, const float* inv_rms,
                                    const void* dres, void* dx, int rows, int cols,
                                    cudaStream_t stream);

}  // namespace ew
}  // namespace mgk
