// Expert-parallel MoE kernels: routing, the dispatch plan, dispatch (token permute fused with
// the all-to-all: every token row is stored straight at its final, expert-sorted position in
// the destination GPU's buffer over NVLink) and combine (the inverse all-to-all fused with the
// un-permute and the gate-weighted sum: every token loads its expert outputs from the GPUs
// that computed them).  Variable per-peer counts make this an all-to-all-v, which the reference
// interface does not have (its all_to_all moves equal chunks, include/megray/communicator.h:75-77).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgk {
namespace moe {

constexpr int kMaxRanks = 8;
constexpr int kMaxExperts = 256;
constexpr int kTopK = 2;
constexpr int kBlockRows = 128;  // expert segments are padded to whole GEMM row blocks

// Top-2 routing: idx[t, k] = expert of slot k, w[t, k] = softmax over the two selected logits;
// counts[e] (+)= number of (token, slot) pairs routed to expert e (counts must be zero before).
cudaError_t launch_route(const float* logits, int tokens, int experts, int* idx, float* w, int* counts,
                         cudaStream_t stream);

// Backward of the gate weights: dlogits[t, e] = d softmax over the chosen pair (zero elsewhere).
cudaError_t launch_route_bwd(const int* idx, const float* w, const float* dw, int tokens, int experts,
                             float* dlogits, cudaStream_t stream);

// Plan (one small block).  counts_all[r][e]: pairs rank r routes to expert e (after an all_gather).
// Experts are owned in contiguous groups of experts/nranks.  Outputs for this rank:
//   send_base[e]    first row, in the owner's buffer, of this rank's tokens for expert e
//   seg_begin[le], seg_end[le]   row range of local expert le in this rank's buffer (end includes
//                                the zero padding up to a multiple of 128)
//   seg_rows[le]    real (unpadded) rows of local expert le
//   block_group[b]  local expert of 128-row block b of this rank's buffer, -1 beyond the last one
//   total[0] = rows in use (padded), total[1] = 1 if any owner's buffer would overflow `capacity`
struct PlanOut {
    int* send_base;
    int* seg_begin;
    int* seg_end;
    int* seg_rows;
    int* block_group;
    int* total;
};
cudaError_t launch_plan(const int* counts_all, int nranks, int rank, int experts, int capacity_rows,
                        PlanOut out, cudaStream_t stream);

// The plan with the count exchange inside the launch.  `counts` are this rank's counts; they
// travel to the peers as flagged 8-byte words through small-message slots of the communicator
// (heap[q] + slot_off + source rank * slot_stride, reserved for this call together with `seq`).
struct PlanExchange {
    char* heap[kMaxRanks];  // every rank's heap as mapped here
    uint64_t slot_off;
    uint64_t slot_stride;
    uint32_t seq;           // this call's flag value (never 0)
    uint64_t timeout_ns;
    int* status;            // communicator status word: MEGRAY_TIMEOUT when a wait runs out
};
cudaError_t launch_plan_exchange(const int* counts, const PlanExchange& x, int nranks, int rank, int experts,
                                 int capacity_rows, PlanOut out, cudaStream_t stream);

// Zero the padding rows [seg_begin+seg_rows, seg_end) of every local expert in `buf`.
cudaError_t launch_zero_pads(void* buf, int row_elems, const int* seg_begin, const int* seg_rows,
                             const int* seg_end, int local_experts, cudaStream_t stream);

struct PeerBufs {
    void* p[kMaxRanks];
};

// Rows at or beyond `capacity_rows` (an owner whose buffer is too small; the plan raises total[1])
// are dropped by dispatch and contribute zero in combine.
// Dispatch.  For every (token t, slot k): row = pos_in[t,k] if pos_in != null, else
// send_base[e] + (a unique slot taken from cursor[e], which must be zero before) and pos_out[t,k] =
// row; then dst[e / local_experts][row, :] = scale * src[t, :], scale = w[t,k] if w != null else 1.
// `experts` is the number of experts the buffers in `dst` own together; an idx entry outside
// [0, experts) drops that (token, slot): pos_out = -1 and nothing else is touched for it.
cudaError_t launch_dispatch(const void* src, int tokens, int row_elems, const int* idx, const float* w,
                            const int* send_base, int* cursor, const int* pos_in, int* pos_out,
                            PeerBufs dst, int experts, int local_experts, int capacity_rows,
                            cudaStream_t stream);

// Combine: out[t, :] = sum_k (w ? w[t,k] : 1) * src[idx[t,k] / local_experts][pos[t,k], :].
cudaError_t launch_combine(void* out, int tokens, int row_elems, const int* idx, const float* w,
                           const int* pos, PeerBufs src, int local_experts, int capacity_rows, cudaStream_t stream);

// Gate gradient: dw[t,k] = dot(dout[t, :], src[owner][pos[t,k], :]).
cudaError_t launch_combine_dw(const void* dout, int tokens, int row_elems, const int* idx, const int* pos,
                              PeerBufs src, int local_experts, int capacity_rows, float* dw, cudaStream_t stream);

}  // namespace moe
}  // namespace mgk
