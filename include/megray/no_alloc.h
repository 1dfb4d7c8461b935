/**
 * MoE token dispatch for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference library.
 *
 * Who needs it: code that runs where a device allocation is impossible or forbidden.  Typical
 * cases are a serving process that has handed all free HBM to its own cache allocator, so that a
 * cudaMalloc made on its behalf fails; a plugin that runs inside another framework's step and is
 * not allowed to touch that framework's allocator; and a latency-critical loop where the implicit
 * device synchronisation of cudaMalloc / cudaFree is unacceptable.  The regular dispatch call
 * (megray_moe_dispatch) expects the caller to supply a zeroed per-expert cursor array; this one
 * needs nothing but the inputs and outputs, because its cursors live in a fixed array inside the
 * library image.
 *
 * What it does: exactly the dispatch of megray_moe_dispatch with fresh row assignment: for every
 * (token t, slot k) it takes the next free row of expert idx[t,k] (send_base[e] + a running
 * count), records it in pos_out[t,k] and stores scale * src[t, :] at that row of the buffer of
 * the rank that owns the expert (scale = w[t,k], or 1 if w is NULL).
 *
 * Layout: routing is top-2.  idx (int32), w (float32, may be NULL) and pos_out (int32) are
 * row-major [tokens, 2] arrays; src is [tokens, row_elems] bf16; send_base has `experts` entries;
 * expert e lives on rank e / local_experts, whose buffer is peer_bufs[e / local_experts]
 * ([capacity_rows, row_elems] bf16).  Tables of any other top-k do not fit this call.
 * An idx entry outside [0, experts) is not an error of the call: that (token, slot) is dropped,
 * its pos_out is -1, and no cursor and no buffer is touched for it.
 *
 * Limits and rules:
 *  - at most MEGRAY_NOALLOC_MAX_EXPERTS experts; a larger `experts` (or nranks > 8, or
 *    experts > nranks * local_experts, or a row length that is not a multiple of 8 elements) is
 *    refused with return value 6 and a message on stderr, and nothing is launched;
 *  - the cursor array (MEGRAY_NOALLOC_MAX_EXPERTS * 4 bytes) is part of the library and stays
 *    resident on every GPU that loads it, until the process exits;
 *  - the first call on each device looks the array's device address up (with that device
 *    current).  Make that first call outside any stream capture;
 *  - every call clears the cursors it uses on `stream` before the kernel, then leaves its counts
 *    behind.  All calls on a device share the one array: two calls that overlap on the GPU
 *    (different streams, no ordering between them) race with each other.  Order them;
 *  - it calls neither cudaMalloc nor cudaFree nor any other allocating routine.
 *
 * Returns 0, 6 (invalid argument / over the limit) or the negated cudaError_t of a failed call.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MEGRAY_NOALLOC_MAX_EXPERTS 256

int megray_moe_dispatch_noalloc(const void* src, int tokens, int row_elems, const int* idx, const float* w,
                                const int* send_base, int experts, int* pos_out, void* const* peer_bufs,
                                int nranks, int local_experts, int capacity_rows, void* stream);

#ifdef __cplusplus
}
#endif
