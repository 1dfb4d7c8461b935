#include "moe.cuh"

#include <cuda_bf16.h>

#include "launch_count.h"

namespace mgk {
namespace moe {

namespace {

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}

// ---------------------------------------------------------------- routing: one warp per token
__global__ void __launch_bounds__(256) route_kernel(const float* __restrict__ logits, int tokens, int experts,
                                                    int* __restrict__ idx, float* __restrict__ w,
                                                    int* __restrict__ counts) {
    __shared__ int hist[kMaxExperts];
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        hist[e] = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int warps_per_block = blockDim.x >> 5;
    for (int t = blockIdx.x * warps_per_block + (threadIdx.x >> 5); t < tokens; t += gridDim.x * warps_per_block) {
        const float* row = logits + static_cast<size_t>(t) * experts;
        float best = -INFINITY, second = -INFINITY;
        int bi = -1, si = -1;
        for (int e = lane; e < experts; e += 32) {
            const float v = row[e];
            if (v > best || (v == best && e < bi)) {
                second = best;
                si = bi;
                best = v;
                bi = e;
            } else if (v > second || (v == second && e < si)) {
                second = v;
                si = e;
            }
        }
        // merge the per-lane (best, second) pairs: ties go to the lower expert index
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o), os = __shfl_xor_sync(0xffffffffu, second, o);
            const int obi = __shfl_xor_sync(0xffffffffu, bi, o), osi = __shfl_xor_sync(0xffffffffu, si, o);
            auto better = [](float a, int ai, float b, int bi2) {
                return a > b || (a == b && ai >= 0 && (bi2 < 0 || ai < bi2));
            };
            if (better(ob, obi, best, bi)) {
                // other's best wins: our best competes with other's second for second place
                if (better(best, bi, os, osi)) {
                    second = best;
                    si = bi;
                } else {
                    second = os;
                    si = osi;
                }
                best = ob;
                bi = obi;
            } else if (better(ob, obi, second, si)) {
                second = ob;
                si = obi;
            }
        }
        if (lane == 0) {
            const float w0 = 1.f / (1.f + __expf(second - best));
            idx[2 * t] = bi;
            idx[2 * t + 1] = si;
            w[2 * t] = w0;
            w[2 * t + 1] = 1.f - w0;
            atomicAdd(&hist[bi], 1);
            atomicAdd(&hist[si], 1);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        if (hist[e])
            atomicAdd(&counts[e], hist[e]);
}

__global__ void __launch_bounds__(256) route_bwd_kernel(const int* __restrict__ idx, const float* __restrict__ w,
                                                        const float* __restrict__ dw, int tokens, int experts,
                                                        float* __restrict__ dlogits) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens)
        return;
    // w0 = sigmoid(l0 - l1), w1 = 1 - w0: d l0 = (dw0 - dw1) * w0 * w1, d l1 = -d l0
    const float g = (dw[2 * t] - dw[2 * t + 1]) * w[2 * t] * w[2 * t + 1];
    float* row = dlogits + static_cast<size_t>(t) * experts;
    for (int e = 0; e < experts; ++e)
        row[e] = 0.f;
    row[idx[2 * t]] = g;
    row[idx[2 * t + 1]] = -g;
}

// ---------------------------------------------------------------- plan: one block
// counts_all[r * experts + e]: pairs rank r routes to expert e (global or shared memory).
__device__ __forceinline__ void plan_body(const int* counts_all, int nranks, int rank, int experts, int capacity_rows,
                                          const PlanOut& out, int* seg_size, int* seg_start, int* before_me,
                                          int* overflow) {
    const int el = experts / nranks;
    if (threadIdx.x == 0)
        *overflow = 0;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        int tot = 0, before = 0;
        for (int r = 0; r < nranks; ++r) {
            const int c = counts_all[r * experts + e];
            if (r < rank)
                before += c;
            tot += c;
        }
        seg_size[e] = tot;
        before_me[e] = before;
    }
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < nranks) {
        // owner `d` lays its local experts out one after the other, each padded to 128 rows
        const int d = threadIdx.x;
        int row = 0;
        for (int le = 0; le < el; ++le) {
            const int e = d * el + le;
            seg_start[e] = row;
            row += (seg_size[e] + kBlockRows - 1) / kBlockRows * kBlockRows;
        }
        if (row > capacity_rows)
            atomicExch(overflow, 1);
        if (d == rank)
            out.total[0] = row;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += blockDim.x)
        out.send_base[e] = seg_start[e] + before_me[e];
    for (int le = threadIdx.x; le < el; le += blockDim.x) {
        const int e = rank * el + le;
        const int padded = (seg_size[e] + kBlockRows - 1) / kBlockRows * kBlockRows;
        out.seg_begin[le] = seg_start[e];
        out.seg_rows[le] = seg_size[e];
        out.seg_end[le] = seg_start[e] + padded;
    }
    const int blocks = capacity_rows / kBlockRows;
    for (int b = threadIdx.x; b < blocks; b += blockDim.x) {
        const int row = b * kBlockRows;
        int g = -1;
        for (int le = 0; le < el; ++le) {
            const int e = rank * el + le;
            const int padded = (seg_size[e] + kBlockRows - 1) / kBlockRows * kBlockRows;
            if (row >= seg_start[e] && row < seg_start[e] + padded)
                g = le;
        }
        out.block_group[b] = g;
    }
    __syncthreads();
    if (threadIdx.x == 0)
        out.total[1] = *overflow;
}

__global__ void __launch_bounds__(256) plan_kernel(const int* __restrict__ counts_all, int nranks, int rank,
                                                   int experts, int capacity_rows, PlanOut out) {
    __shared__ int seg_size[kMaxExperts];   // rows of expert e over all source ranks
    __shared__ int seg_start[kMaxExperts];  // first row of expert e inside its owner's buffer
    __shared__ int before_me[kMaxExperts];  // rows of expert e from ranks below this one
    __shared__ int overflow;
    plan_body(counts_all, nranks, rank, experts, capacity_rows, out, seg_size, seg_start, before_me, &overflow);
}

// The same plan with the exchange of the counts inside the launch: every rank stores its counts
// into the peers' small-message slots as 8-byte {count, sequence number} words and polls its own
// slots until every word carries this call's sequence number (no barrier, no separate all_gather).
__global__ void __launch_bounds__(256) plan_exchange_kernel(const int* __restrict__ counts, PlanExchange x, int nranks,
                                                            int rank, int experts, int capacity_rows, PlanOut out) {
    __shared__ int seg_size[kMaxExperts];
    __shared__ int seg_start[kMaxExperts];
    __shared__ int before_me[kMaxExperts];
    __shared__ int overflow;
    __shared__ int all[kMaxRanks * kMaxExperts];
    __shared__ int failed;
    if (threadIdx.x == 0)
        failed = 0;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) {
        const int c = counts[e];
        all[rank * experts + e] = c;
        for (int qq = 1; qq < nranks; ++qq) {
            const int q = (rank + qq) % nranks;
            char* slot = x.heap[q] + x.slot_off + static_cast<uint64_t>(rank) * x.slot_stride + static_cast<uint64_t>(e) * 8;
            asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(slot), "r"(static_cast<uint32_t>(c)), "r"(x.seq)
                         : "memory");
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (nranks - 1) * experts; i += blockDim.x) {
        const int q = (rank + 1 + i / experts) % nranks, e = i % experts;
        const char* slot = x.heap[rank] + x.slot_off + static_cast<uint64_t>(q) * x.slot_stride + static_cast<uint64_t>(e) * 8;
        uint32_t v = 0, f = 0, spins = 0;
        unsigned long long t0 = 0;
        for (;;) {
            asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v), "=r"(f) : "l"(slot) : "memory");
            if (f == x.seq)
                break;
            if ((++spins & 255) == 0) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0)
                    t0 = now;
                else if (now - t0 > x.timeout_ns) {
                    if (x.status != nullptr)
                        atomicCAS(x.status, 0, 12);  // MEGRAY_TIMEOUT
                    failed = 1;
                    break;
                }
            }
        }
        all[q * experts + e] = static_cast<int>(v);
    }
    __syncthreads();
    if (failed)
        return;
    plan_body(all, nranks, rank, experts, capacity_rows, out, seg_size, seg_start, before_me, &overflow);
}

__global__ void __launch_bounds__(256) zero_pads_kernel(uint4* __restrict__ buf, int row_vecs,
                                                        const int* __restrict__ seg_begin,
                                                        const int* __restrict__ seg_rows,
                                                        const int* __restrict__ seg_end) {
    const int le = blockIdx.y;
    const int first = seg_begin[le] + seg_rows[le], last = seg_end[le];
    const uint4 z = make_uint4(0, 0, 0, 0);
    for (int r = first + blockIdx.x; r < last; r += gridDim.x)
        for (int v = threadIdx.x; v < row_vecs; v += blockDim.x)
            buf[static_cast<size_t>(r) * row_vecs + v] = z;
}

// ---------------------------------------------------------------- dispatch: one warp per token
// The token's row is read once, eight 16-byte vectors per lane at a time (all loads issued
// before the first store), and stored to the rows of both of its experts.
__global__ void __launch_bounds__(256) dispatch_kernel(const uint4* __restrict__ src, int tokens, int row_vecs,
                                                       const int* __restrict__ idx, const float* __restrict__ w,
                                                       const int* __restrict__ send_base, int* __restrict__ cursor,
                                                       const int* __restrict__ pos_in, int* __restrict__ pos_out,
                                                       PeerBufs dst, int experts, int local_experts,
                                                       int capacity) {
    static_assert(kTopK == 2, "the dispatch kernel stores each token to two experts");
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < tokens; t += gridDim.x * wpb) {
        const int i0 = t * kTopK;
        const int e0 = idx[i0], e1 = idx[i0 + 1];
        // an expert id that no rank owns names no cursor and no buffer: the (token, slot) is dropped
        const bool in0 = static_cast<unsigned>(e0) < static_cast<unsigned>(experts);
        const bool in1 = static_cast<unsigned>(e1) < static_cast<unsigned>(experts);
        // The first vectors of the row are requested before the row positions are known: taking a
        // position is an atomic whose round trip would otherwise sit in front of every row's loads.
        constexpr int U = 8;
        const uint4* s = src + static_cast<size_t>(t) * row_vecs;
        uint4 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (lane + 32 * u < row_vecs)
                x[u] = __ldg(s + lane + 32 * u);
        int row0, row1;
        if (pos_in != nullptr) {
            row0 = pos_in[i0];
            row1 = pos_in[i0 + 1];
        } else {
            row0 = row1 = -1;
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
        }
        // a full owner buffer (the plan has raised the overflow flag) drops the row
        const bool ok0 = in0 && row0 >= 0 && row0 < capacity, ok1 = in1 && row1 >= 0 && row1 < capacity;
        if (!ok0 && !ok1)
            continue;
        const float s0 = w != nullptr ? w[i0] : 1.f, s1 = w != nullptr ? w[i0 + 1] : 1.f;
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
        for (int v0 = lane; v0 < row_vecs; v0 += 32 * U) {
            if (v0 != lane) {  // (the first batch is already in registers)
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (v0 + 32 * u < row_vecs)
                        x[u] = __ldg(s + v0 + 32 * u);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int v = v0 + 32 * u;
                if (v < row_vecs) {
                    if (ok0)
                        d0[v] = w != nullptr ? scaled(x[u], s0) : x[u];
                    if (ok1)
                        d1[v] = w != nullptr ? scaled(x[u], s1) : x[u];
                }
            }
        }
    }
}

// ---------------------------------------------------------------- combine: one warp per token
__global__ void __launch_bounds__(256) combine_kernel(uint4* __restrict__ out, int tokens, int row_vecs,
                                                      const int* __restrict__ idx, const float* __restrict__ w,
                                                      const int* __restrict__ pos, PeerBufs src, int local_experts, int capacity) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (int t = blockIdx.x * wpb + (threadIdx.x >> 5); t < tokens; t += gridDim.x * wpb) {
        const int e0 = idx[2 * t], e1 = idx[2 * t + 1];
        float w0 = w != nullptr ? w[2 * t] : 1.f, w1 = w != nullptr ? w[2 * t + 1] : 1.f;
        const int p0 = pos[2 * t], p1 = pos[2 * t + 1];
        // dropped at dispatch (full owner buffer, or an expert id nobody owns): contributes nothing
        const unsigned owned = static_cast<unsigned>(kMaxRanks * local_experts);
        const bool ok0 = p0 >= 0 && p0 < capacity && static_cast<unsigned>(e0) < owned;
        const bool ok1 = p1 >= 0 && p1 < capacity && static_cast<unsigned>(e1) < owned;
        if (!ok0)
            w0 = 0.f;
        if (!ok1)
            w1 = 0.f;
        const uint4* a = ok0 ? static_cast<const uint4*>(src.p[e0 / local_experts]) + static_cast<size_t>(p0) * row_vecs : nullptr;
        const uint4* b = ok1 ? static_cast<const uint4*>(src.p[e1 / local_experts]) + static_cast<size_t>(p1) * row_vecs : nullptr;
        uint4* o = out + static_cast<size_t>(t) * row_vecs;
        // four vectors of each row per lane and iteration: eight (possibly remote) loads in flight
        constexpr int U = 4;
        for (int v0 = lane; v0 < row_vecs; v0 += 32 * U) {
            uint4 x[U], y[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (v0 + 32 * u < row_vecs) {
                    x[u] = ok0 ? __ldcg(a + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
                    y[u] = ok1 ? __ldcg(b + v0 + 32 * u) : make_uint4(0, 0, 0, 0);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (v0 + 32 * u < row_vecs) {
                    uint4 r;
                    r.x = pack(w0 * lo(x[u].x) + w1 * lo(y[u].x), w0 * hi(x[u].x) + w1 * hi(y[u].x));
                    r.y = pack(w0 * lo(x[u].y) + w1 * lo(y[u].y), w0 * hi(x[u].y) + w1 * hi(y[u].y));
                    r.z = pack(w0 * lo(x[u].z) + w1 * lo(y[u].z), w0 * hi(x[u].z) + w1 * hi(y[u].z));
                    r.w = pack(w0 * lo(x[u].w) + w1 * lo(y[u].w), w0 * hi(x[u].w) + w1 * hi(y[u].w));
                    o[v0 + 32 * u] = r;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(256) combine_dw_kernel(const uint4* __restrict__ dout, int tokens, int row_vecs,
                                                         const int* __restrict__ idx, const int* __restrict__ pos,
                                                         PeerBufs src, int local_experts, int capacity, float* __restrict__ dw) {
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    const int pairs = tokens * kTopK;
    for (int i = blockIdx.x * wpb + (threadIdx.x >> 5); i < pairs; i += gridDim.x * wpb) {
        if (pos[i] < 0 || pos[i] >= capacity ||
            static_cast<unsigned>(idx[i]) >= static_cast<unsigned>(kMaxRanks * local_experts)) {
            if (lane == 0)
                dw[i] = 0.f;
            continue;
        }
        const uint4* g = dout + static_cast<size_t>(i / kTopK) * row_vecs;
        const uint4* y = static_cast<const uint4*>(src.p[idx[i] / local_experts]) + static_cast<size_t>(pos[i]) * row_vecs;
        float acc = 0.f;
        for (int v = lane; v < row_vecs; v += 32) {
            const uint4 a = g[v], b = __ldcg(y + v);
            acc += lo(a.x) * lo(b.x) + hi(a.x) * hi(b.x) + lo(a.y) * lo(b.y) + hi(a.y) * hi(b.y) +
                   lo(a.z) * lo(b.z) + hi(a.z) * hi(b.z) + lo(a.w) * lo(b.w) + hi(a.w) * hi(b.w);
        }
        for (int o = 16; o > 0; o >>= 1)
            acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0)
            dw[i] = acc;
    }
}

int blocks_for(int items_per_block, long items) {
    long b = (items + items_per_block - 1) / items_per_block;
    if (b < 1)
        b = 1;
    if (b > 148 * 8)
        b = 148 * 8;
    return static_cast<int>(b);
}

}  // namespace

cudaError_t launch_route(const float* logits, int tokens, int experts, int* idx, float* w, int* counts,
                         cudaStream_t stream) {
    if (tokens <= 0 || experts < 2 || experts > kMaxExperts)
        return cudaErrorInvalidValue;
    route_kernel<<<blocks_for(8, tokens), 256, 0, stream>>>(logits, tokens, experts, idx, w, counts);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_route_bwd(const int* idx, const float* w, const float* dw, int tokens, int experts,
                             float* dlogits, cudaStream_t stream) {
    if (tokens <= 0)
        return cudaErrorInvalidValue;
    route_bwd_kernel<<<(tokens + 255) / 256, 256, 0, stream>>>(idx, w, dw, tokens, experts, dlogits);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_plan(const int* counts_all, int nranks, int rank, int experts, int capacity_rows,
                        PlanOut out, cudaStream_t stream) {
    if (nranks < 1 || nranks > kMaxRanks || experts % nranks || experts > kMaxExperts ||
        capacity_rows % kBlockRows)
        return cudaErrorInvalidValue;
    plan_kernel<<<1, 256, 0, stream>>>(counts_all, nranks, rank, experts, capacity_rows, out);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_plan_exchange(const int* counts, const PlanExchange& x, int nranks, int rank, int experts,
                                 int capacity_rows, PlanOut out, cudaStream_t stream) {
    if (nranks < 1 || nranks > kMaxRanks || experts % nranks || experts > kMaxExperts || capacity_rows % kBlockRows ||
        x.seq == 0 || static_cast<uint64_t>(experts) * 8 > x.slot_stride)
        return cudaErrorInvalidValue;
    plan_exchange_kernel<<<1, 256, 0, stream>>>(counts, x, nranks, rank, experts, capacity_rows, out);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_zero_pads(void* buf, int row_elems, const int* seg_begin, const int* seg_rows,
                             const int* seg_end, int local_experts, cudaStream_t stream) {
    if (row_elems % 8 || local_experts < 1)
        return cudaErrorInvalidValue;
    zero_pads_kernel<<<dim3(16, local_experts), 256, 0, stream>>>(static_cast<uint4*>(buf), row_elems / 8, seg_begin,
                                                                  seg_rows, seg_end);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_dispatch(const void* src, int tokens, int row_elems, const int* idx, const float* w,
                            const int* send_base, int* cursor, const int* pos_in, int* pos_out, PeerBufs dst,
                            int experts, int local_experts, int capacity, cudaStream_t stream) {
    if (tokens <= 0 || row_elems % 8 || local_experts < 1 || experts < 1 ||
        experts > kMaxRanks * local_experts)
        return cudaErrorInvalidValue;
    dispatch_kernel<<<blocks_for(8, tokens), 256, 0, stream>>>(
            static_cast<const uint4*>(src), tokens, row_elems / 8, idx, w, send_base, cursor, pos_in, pos_out, dst,
            experts, local_experts, capacity);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_combine(void* out, int tokens, int row_elems, const int* idx, const float* w, const int* pos,
                           PeerBufs src, int local_experts, int capacity, cudaStream_t stream) {
    if (tokens <= 0 || row_elems % 8 || local_experts < 1)
        return cudaErrorInvalidValue;
    combine_kernel<<<blocks_for(8, tokens), 256, 0, stream>>>(static_cast<uint4*>(out), tokens, row_elems / 8, idx, w,
                                                              pos, src, local_experts, capacity);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_combine_dw(const void* dout, int tokens, int row_elems, const int* idx, const int* pos,
                              PeerBufs src, int local_experts, int capacity, float* dw, cudaStream_t stream) {
    if (tokens <= 0 || row_elems % 8 || local_experts < 1)
        return cudaErrorInvalidValue;
    combine_dw_kernel<<<blocks_for(8, static_cast<long>(tokens) * kTopK), 256, 0, stream>>>(
            static_cast<const uint4*>(dout), tokens, row_elems / 8, idx, pos, src, local_experts, capacity, dw);
    count_launch();
    return cudaGetLastError();
}

}  // namespace moe
}  // namespace mgk
