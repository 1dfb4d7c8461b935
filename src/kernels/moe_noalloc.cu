// megray_moe_dispatch_noalloc: MoE dispatch whose per-expert cursors live in a fixed device
// array of this library instead of caller-provided memory (see include/megray/no_alloc.h for
// who needs that and for the rules of use).  Nothing here allocates.
#include "megray/no_alloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdio.h>

#include <mutex>

#include "launch_count.h"

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

// One warp per (token, slot): take a row of the expert's segment, remember it, store the row.
__global__ void __launch_bounds__(256)
        dispatch_noalloc_kernel(const uint4* __restrict__ src, int tokens, int row_vecs, const int* __restrict__ idx,
                                const float* __restrict__ w, const int* __restrict__ send_base,
                                int* __restrict__ cursor, int* __restrict__ pos_out, Peers dst, int local_experts,
                                int capacity) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const int pairs = tokens * 2;
    for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < pairs; i += gridDim.x * wpb) {
        const int e = idx[i];
        int row = 0;
        if (lane == 0) {
            row = send_base[e] + atomicAdd(&cursor[e], 1);
            pos_out[i] = row;
        }
        row = __shfl_sync(0xffffffffu, row, 0);
        if (row < 0 || row >= capacity)
            continue;  // the owner's buffer is full: the row is dropped, as in the regular dispatch
        const float scale = w != nullptr ? w[i] : 1.f;
        const uint4* s = src + static_cast<size_t>(i / 2) * row_vecs;
        uint4* d = static_cast<uint4*>(dst.p[e / local_experts]) + static_cast<size_t>(row) * row_vecs;
        for (int v = lane; v < row_vecs; v += 32) {
            uint4 x = s[v];
            if (w != nullptr) {
                x.x = pack(lo(x.x) * scale, hi(x.x) * scale);
                x.y = pack(lo(x.y) * scale, hi(x.y) * scale);
                x.z = pack(lo(x.z) * scale, hi(x.z) * scale);
                x.w = pack(lo(x.w) * scale, hi(x.w) * scale);
            }
            d[v] = x;
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
    long blocks = (static_cast<long>(tokens) * 2 + 7) / 8;
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    dispatch_noalloc_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(
            static_cast<const uint4*>(src), tokens, row_elems / 8, idx, w, send_base, cursor, pos_out, dst,
            local_experts, capacity_rows);
    mgk::count_launch();
    e = cudaGetLastError();
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
