// Host-side elementwise reduction for every numeric dtype: the arithmetic of
// the host backend and the oracle that device kernels are tested against.
//
// The reference's host reduction (src/shm/utils.cpp:16-69) covers six dtypes;
// this one covers all ten numeric ones.  fp16 / bf16 inputs are widened to
// fp32, combined in the order given, and rounded once at the end
// (round-to-nearest-even), which is also what the device kernels do.
// Integers wrap modulo 2^width.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include "megray/types.h"

namespace MegRay {
namespace host {

/** out[i] = op(in[0][i], in[1][i], ... in[n_in-1][i]) for i < len; out may alias any input.
 *  Returns MEGRAY_INVALID_ARGUMENT for MEGRAY_CHAR or unknown enums. */
Status cpu_reduce_n(const void* const* in, int n_in, void* out, size_t len, DType dtype,
                    ReduceOp op);

/** Two-input form: out = op(a, b). */
Status cpu_reduce(const void* a, const void* b, void* out, size_t len, DType dtype, ReduceOp op);

/** out[i] = cast<out_dtype>(scale * op-reduction of the inputs): the host model of the fused
 *  scale/cast all_reduce. Float dtypes only (fp16, bf16, fp32, fp64). */
Status cpu_reduce_scale_cast(const void* const* in, int n_in, DType in_dtype, void* out,
                             DType out_dtype, size_t len, ReduceOp op, double scale);

float half_to_float(uint16_t h);
uint16_t float_to_half(float f);
float bf16_to_float(uint16_t b);
uint16_t float_to_bf16(float f);

}  // namespace host
}  // namespace MegRay
