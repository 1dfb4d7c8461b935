// C entry points of the MoE kernels (see include/megray/c_api.h).
#include <memory>

#include "kernels/moe.cuh"
#include "megray/c_api.h"
#include "megray/communicator.h"
#include "megray/fused.h"

namespace {
int rc(cudaError_t e) { return e == cudaSuccess ? 0 : -static_cast<int>(e); }
mgk::moe::PeerBufs bufs(void* const* p, int n) {
    mgk::moe::PeerBufs b{};
    for (int i = 0; i < n && i < mgk::moe::kMaxRanks; ++i)
        b.p[i] = p[i];
    return b;
}
cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
struct CommBoxView {  // layout of the handle made by megray_comm_new (capi/comm_c.cpp)
    std::shared_ptr<MegRay::Communicator> comm;
};
}  // namespace

extern "C" {

int megray_moe_route(const float* logits, int tokens, int experts, int* idx, float* w, int* counts, void* stream) {
    return rc(mgk::moe::launch_route(logits, tokens, experts, idx, w, counts, S(stream)));
}
int megray_moe_route_bwd(const int* idx, const float* w, const float* dw, int tokens, int experts, float* dlogits,
                         void* stream) {
    return rc(mgk::moe::launch_route_bwd(idx, w, dw, tokens, experts, dlogits, S(stream)));
}
int megray_moe_plan(const int* counts_all, int nranks, int rank, int experts, int capacity_rows, int* send_base,
                    int* seg_begin, int* seg_end, int* seg_rows, int* block_group, int* total, void* stream) {
    mgk::moe::PlanOut o{send_base, seg_begin, seg_end, seg_rows, block_group, total};
    return rc(mgk::moe::launch_plan(counts_all, nranks, rank, experts, capacity_rows, o, S(stream)));
}
int megray_moe_plan_exchange(void* comm, const int* counts, int experts, int capacity_rows, int* send_base,
                             int* seg_begin, int* seg_end, int* seg_rows, int* block_group, int* total, void* stream) {
    if (comm == nullptr)
        return 6;
    MegRay::Communicator* c = static_cast<CommBoxView*>(comm)->comm.get();
    MegRay::NvlInterface* nvl = MegRay::as_nvl(c);
    if (nvl == nullptr)
        return 7;
    const MegRay::Status st = nvl->fused_begin(stream);
    if (st != MegRay::MEGRAY_OK)
        return st;
    mgk::moe::PlanExchange x{};
    const int n = static_cast<int>(c->nranks());
    for (int q = 0; q < n && q < mgk::moe::kMaxRanks; ++q)
        x.heap[q] = static_cast<char*>(nvl->heap_base(static_cast<uint32_t>(q)));
    size_t off = 0, stride = 0;
    nvl->ll_ticket(&x.seq, &off, &stride);
    x.slot_off = off;
    x.slot_stride = stride;
    x.timeout_ns = nvl->device_timeout_ns();
    x.status = nvl->status_word();
    mgk::moe::PlanOut o{send_base, seg_begin, seg_end, seg_rows, block_group, total};
    const int r = rc(mgk::moe::launch_plan_exchange(counts, x, n, static_cast<int>(c->rank()), experts, capacity_rows, o,
                                                    S(stream)));
    if (r == 0)
        nvl->fused_end(stream);
    return r;
}
int megray_moe_zero_pads(void* buf, int row_elems, const int* seg_begin, const int* seg_rows, const int* seg_end,
                         int local_experts, void* stream) {
    return rc(mgk::moe::launch_zero_pads(buf, row_elems, seg_begin, seg_rows, seg_end, local_experts, S(stream)));
}
int megray_moe_dispatch(const void* src, int tokens, int row_elems, const int* idx, const float* w,
                        const int* send_base, int* cursor, const int* pos_in, int* pos_out, void* const* peer_bufs,
                        int nranks, int local_experts, int capacity_rows, void* stream) {
    if (nranks < 1 || nranks > mgk::moe::kMaxRanks || local_experts < 1)
        return 6;
    return rc(mgk::moe::launch_dispatch(src, tokens, row_elems, idx, w, send_base, cursor, pos_in, pos_out,
                                        bufs(peer_bufs, nranks), nranks * local_experts, local_experts,
                                        capacity_rows, S(stream)));
}
int megray_moe_combine(void* out, int tokens, int row_elems, const int* idx, const float* w, const int* pos,
                       void* const* peer_bufs, int nranks, int local_experts, int capacity_rows, void* stream) {
    if (nranks < 1 || nranks > mgk::moe::kMaxRanks)
        return 6;
    return rc(mgk::moe::launch_combine(out, tokens, row_elems, idx, w, pos, bufs(peer_bufs, nranks), local_experts,
                                       capacity_rows, S(stream)));
}
int megray_moe_combine_dw(const void* dout, int tokens, int row_elems, const int* idx, const int* pos,
                          void* const* peer_bufs, int nranks, int local_experts, int capacity_rows, float* dw, void* stream) {
    if (nranks < 1 || nranks > mgk::moe::kMaxRanks)
        return 6;
    return rc(mgk::moe::launch_combine_dw(dout, tokens, row_elems, idx, pos, bufs(peer_bufs, nranks), local_experts,
                                          capacity_rows, dw, S(stream)));
}

}  // extern "C"
