// megray_moe_dispatch_noalloc: MoE dispatch whose per-expert cursors live in a fixed device
// array of this library instead of caller-provided memory (see include/megray/no_alloc.h for
// who needs that and for the rules of use).  Nothing here allocates.
#include "megray/no_alloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "launch_count.h"
#include "moe.cuh"

namespace {

// The scratch: one running count per expert.  It is resident on every GPU that loads the
// library.  In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) int g_dispatch_cursor[MEGRAY_NOALLOC_MAX_EXPERTS];

constexpr int kMaxDevices = 64;
constexpr int kMaxRanks = 8;
std::mutex g_mu;
int* g_cursor_addr[kMaxDevices] = {nullptr};  // device address of the array, per device ordinal

struct Peers {
    void* p[kMaxRanks];
};

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// One warp per token: both of its experts take the next row of their segments, the token's row is
// read once and stored to both.  idx, w and pos_out are [tokens, 2] (top-2 routing, as in moe.cu).
// An expert id outside [0, experts) names no cursor and no owner: that (token, slot) is dropped,
// pos_out = -1, and nothing else is touched.
__global__ void __launch_bounds__(256)
        dispatch_noalloc_kernel(const uint4* __restrict__ src, int tokens, int row_vecs, const int* __restrict__ idx,
                                const float* __restrict__ w, const int* __restrict__ send_base,
                                int* __restrict__ cursor, int* __restrict__ pos_out, Peers dst, int experts,
                                int local_experts, int capacity) {
    static_assert(mgk::moe::kTopK == 2, "the kernel stores each token to two experts");
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < tokens; t += gridDim.x * wpb) {
        const int i0 = 2 * t;
        const int e0 = idx[i0], e1 = idx[i0 + 1];
        const bool in0 = static_cast<unsigned>(e0) < static_cast<unsigned>(experts);
        const bool in1 = static_cast<unsigned>(e1) < static_cast<unsigned>(experts);
        int row0 = -1, row1 = -1;
        if (lane == 0) {
            if (in0)
                row0 = send_base[e0] + atomicAdd(&cursor[e0], 1);
            if (in1)
                row1 = send_base[e1] + atomicAdd(&cursor[e1], 1);
            pos_out[i0] = row0;
            pos_out[i0 + 1] = row1;
        }
        row0 = __shfl_sync(0xffffffffu, row0, 0);
        row1 = __shfl_sync(0xffffffffu, row1, 0);
        // a full owner buffer drops the row, as in the regular dispatch
        const bool ok0 = in0 && row0 >= 0 && row0 < capacity, ok1 = in1 && row1 >= 0 && row1 < capacity;
        if (!ok0 && !ok1)
            continue;
        const float s0 = w != nullptr ? w[i0] : 1.f, s1 = w != nullptr ? w[i0 + 1] : 1.f;
        const uint4* s = src + static_cast<size_t>(t) * row_vecs;
        uint4* d0 = ok0 ? static_cast<uint4*>(dst.p[e0 / local_experts]) + static_cast<size_t>(row0) * row_vecs : nullptr;
        uint4* d1 = ok1 ? static_cast<uint4*>(dst.p[e1 / local_experts]) + static_cast<size_t>(row1) * row_vecs : nullptr;
        auto scaled = [](const uint4& x, float f) {
            uint4 y;
            y.x = pack(lo(x.x) * f, hi(x.x) * f);
            y.y = pack(lo(x.y) * f, hi(x.y) * f);
            y.z = pack(lo(x.z) * f, hi(x.z) * f);
            y.w = pack(lo(x.w) * f, hi(x.w) * f);
            return y;
        };
        for (int v = lane; v < row_vecs; v += 32) {
            const uint4 x = s[v];
            if (ok0)
                d0[v] = w != nullptr ? scaled(x, s0) : x;
            if (ok1)
                d1[v] = w != nullptr ? scaled(x, s1) : x;
        }
    }
}

// Device address of the cursor array on the current device; looked up once per device.
cudaError_t cursor_address(int** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess)
        return e;
    if (dev < 0 || dev >= kMaxDevices)
        return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_cursor_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_dispatch_cursor);
        if (e != cudaSuccess)
            return e;
        g_cursor_addr[dev] = static_cast<int*>(p);
    }
    *out = g_cursor_addr[dev];
    return cudaSuccess;
}

}  // namespace

extern "C" int megray_moe_dispatch_noalloc(const void* src, int tokens, int row_elems, const int* idx,
                                           const float* w, const int* send_base, int experts, int* pos_out,
                                           void* const* peer_bufs, int nranks, int local_experts,
                                           int capacity_rows, void* stream) {
    if (experts > MEGRAY_NOALLOC_MAX_EXPERTS) {
        fprintf(stderr,
                "megray_moe_dispatch_noalloc: %d experts exceed the built-in cursor array of %d; use "
                "megray_moe_dispatch with a caller-provided cursor array instead\n",
                experts, MEGRAY_NOALLOC_MAX_EXPERTS);
        return 6;
    }
    if (src == nullptr || idx == nullptr || send_base == nullptr || pos_out == nullptr || peer_bufs == nullptr ||
        tokens <= 0 || experts < 1 || row_elems <= 0 || row_elems % 8 || nranks < 1 || nranks > kMaxRanks ||
        local_experts < 1 || capacity_rows < 0) {
        fprintf(stderr, "megray_moe_dispatch_noalloc: invalid argument (row length must be a multiple of 8 "
                        "elements, 1..8 ranks, non-null inputs and outputs)\n");
        return 6;
    }
    if (static_cast<long>(experts) > static_cast<long>(nranks) * local_experts) {
        fprintf(stderr, "megray_moe_dispatch_noalloc: %d experts need %d owners of %d experts each, but only %d "
                        "peer buffers were given\n",
                experts, (experts + local_experts - 1) / local_experts, local_experts, nranks);
        return 6;
    }
    int* cursor = nullptr;
    cudaError_t e = cursor_address(&cursor);
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // the array keeps the previous call's counts: the cursors this call uses start from zero
    e = cudaMemsetAsync(cursor, 0, static_cast<size_t>(experts) * sizeof(int), s);
    if (e != cudaSuccess)
        return -static_cast<int>(e);
    Peers dst{};
    for (int q = 0; q < nranks; ++q)
        dst.p[q] = peer_bufs[q];
    long blocks = (static_cast<long>(tokens) + 7) / 8;
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    dispatch_noalloc_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(
            static_cast<const uint4*>(src), tokens, row_elems / 8, idx, w, send_base, cursor, pos_out, dst,
            experts, local_experts, capacity_rows);
    mgk::count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
