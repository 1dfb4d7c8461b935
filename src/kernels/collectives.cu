// Native collective kernels over NVLink peer memory (see collectives.cuh for the protocol).
#include "collectives.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "launch_count.h"
#include "ptx_sm100.cuh"

namespace mgk {
namespace coll {

using namespace mgk::ptx;
using MegRay::DType;
using MegRay::ReduceOp;

namespace {

constexpr int kStatusTimeout = 12;  // MegRay::MEGRAY_TIMEOUT

__device__ __forceinline__ uint64_t round_up_u64(uint64_t v, uint64_t a) {
    return (v + a - 1) / a * a;
}

// ------------------------------------------------------------------ barrier
// One flag word per (CTA, peer) in every rank's pad.  Returns false when a wait ran out.
__device__ __forceinline__ bool cta_barrier(const CommonArgs& c, uint32_t target) {
    __syncthreads();
    int ok = 1;
    if (threadIdx.x < static_cast<unsigned>(c.nranks)) {
        const int q = threadIdx.x;
        uint32_t* at_peer = reinterpret_cast<uint32_t*>(c.peers.heap[q] + c.flag_off) +
                            blockIdx.x * kMaxRanks + c.rank;
        st_release_sys(at_peer, target);
        const uint32_t* mine = reinterpret_cast<const uint32_t*>(c.peers.heap[c.rank] + c.flag_off) +
                               blockIdx.x * kMaxRanks + q;
        uint32_t spins = 0;
        uint64_t t0 = 0;
        while (static_cast<int32_t>(ld_acquire_sys(mine) - target) < 0) {
            if ((++spins & 63) == 0) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0)
                    t0 = now;
                else if (now - t0 > c.timeout_ns) {
                    ok = 0;
                    if (c.status != nullptr)
                        atomicCAS(c.status, 0, kStatusTimeout);
                    break;
                }
            }
        }
    }
    return __syncthreads_and(ok) != 0;
}

// ------------------------------------------------------------------ copies
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}

// CTA-cooperative byte copy for any alignment.  Vector (16 B) body when source and
// destination are equally aligned, else 4-byte or 1-byte units.
__device__ __forceinline__ void cta_copy(char* dst, const char* src, uint64_t nbytes) {
    if (nbytes == 0)
        return;
    const uintptr_t da = reinterpret_cast<uintptr_t>(dst), sa = reinterpret_cast<uintptr_t>(src);
    const unsigned tid = threadIdx.x, nth = blockDim.x;
    if (((da ^ sa) & 15) == 0) {
        uint64_t head = (16 - (da & 15)) & 15;
        if (head > nbytes)
            head = nbytes;
        for (uint64_t i = tid; i < head; i += nth)
            dst[i] = src[i];
        const uint64_t body = (nbytes - head) / 16;
        const uint4* s4 = reinterpret_cast<const uint4*>(src + head);
        uint4* d4 = reinterpret_cast<uint4*>(dst + head);
        uint64_t i = tid;
        // eight, then four, independent 16-byte loads in flight per thread: a peer load takes a
        // few microseconds, and the link only fills with megabytes in flight
        for (; i + 7ull * nth < body; i += 8ull * nth) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = __ldcg(s4 + i + static_cast<uint64_t>(u) * nth);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                d4[i + static_cast<uint64_t>(u) * nth] = v[u];
        }
        for (; i + 3ull * nth < body; i += 4ull * nth) {
            uint4 a = __ldcg(s4 + i), b = __ldcg(s4 + i + nth), c2 = __ldcg(s4 + i + 2ull * nth),
                  d = __ldcg(s4 + i + 3ull * nth);
            d4[i] = a;
            d4[i + nth] = b;
            d4[i + 2ull * nth] = c2;
            d4[i + 3ull * nth] = d;
        }
        for (; i < body; i += nth)
            d4[i] = __ldcg(s4 + i);
        const uint64_t done = head + body * 16;
        for (uint64_t k = done + tid; k < nbytes; k += nth)
            dst[k] = src[k];
    } else if (((da | sa | nbytes) & 3) == 0) {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
        uint32_t* d = reinterpret_cast<uint32_t*>(dst);
        for (uint64_t i = tid; i < nbytes / 4; i += nth)
            d[i] = __ldcg(s + i);
    } else {
        for (uint64_t i = tid; i < nbytes; i += nth)
            dst[i] = src[i];
    }
}

// ------------------------------------------------------------------ arithmetic
template <typename T>
struct Acc {
    using type = T;
};
template <>
struct Acc<__half> {
    using type = float;
};
template <>
struct Acc<__nv_bfloat16> {
    using type = float;
};

template <typename T>
__device__ __forceinline__ typename Acc<T>::type widen(T v) {
    return v;
}
template <>
__device__ __forceinline__ float widen<__half>(__half v) {
    return __half2float(v);
}
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

template <typename To, typename A>
__device__ __forceinline__ To narrow(A v) {
    return static_cast<To>(v);
}
template <>
__device__ __forceinline__ __half narrow<__half, float>(float v) {
    return __float2half_rn(v);
}
template <>
__device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) {
    return __float2bfloat16_rn(v);
}

template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b) {
    if (OP == MegRay::MEGRAY_SUM)
        return static_cast<A>(a + b);
    if (OP == MegRay::MEGRAY_MAX)
        return a > b ? a : b;
    return a < b ? a : b;
}

template <typename A>
struct IsFloatAcc {
    static constexpr bool value = false;
};
template <>
struct IsFloatAcc<float> {
    static constexpr bool value = true;
};
template <>
struct IsFloatAcc<double> {
    static constexpr bool value = true;
};

// out[0..n) = cast(scale * op over k of slot_k[0..n)), slots `slot_stride` bytes apart.
// `slots` and `out` are 16-byte aligned (staging memory); n is in elements.
template <typename Tin, typename Tout, int OP>
__device__ __forceinline__ void cta_reduce_slots(const char* slots, uint64_t slot_stride, int nslots,
                                                 char* out, uint64_t n, float scale) {
    using A = typename Acc<Tin>::type;
    constexpr int V = 16 / sizeof(Tin);
    const unsigned tid = threadIdx.x, nth = blockDim.x;
    const uint64_t nvec = n / V;
    const bool do_scale = IsFloatAcc<A>::value && OP == MegRay::MEGRAY_SUM && scale != 1.0f;
    for (uint64_t i = tid; i < nvec; i += nth) {
        // all slots' loads are issued before the first use
        uint4 raw[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)
            if (s < nslots)
                raw[s] = ld_cg_v4(slots + s * slot_stride + i * 16);
        A acc[V];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
            if (s < nslots) {
                const Tin* e = reinterpret_cast<const Tin*>(&raw[s]);
#pragma unroll
                for (int k = 0; k < V; ++k)
                    acc[k] = s == 0 ? widen<Tin>(e[k]) : combine<OP, A>(acc[k], widen<Tin>(e[k]));
            }
        }
        if (do_scale) {
#pragma unroll
            for (int k = 0; k < V; ++k)
                acc[k] = static_cast<A>(acc[k] * static_cast<A>(scale));
        }
        Tout o[V];
#pragma unroll
        for (int k = 0; k < V; ++k)
            o[k] = narrow<Tout, A>(acc[k]);
        // V * sizeof(Tout) bytes, written as 16-byte pieces
        constexpr int OB = V * sizeof(Tout);
        char* dst = out + i * OB;
        if (OB >= 16) {
#pragma unroll
            for (int b = 0; b < OB / 16; ++b)
                reinterpret_cast<uint4*>(dst)[b] = reinterpret_cast<const uint4*>(o)[b];
        } else {  // narrowing cast (e.g. fp32 -> bf16): 8 bytes
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
        }
    }
    // element tail
    for (uint64_t i = nvec * V + tid; i < n; i += nth) {
        A acc = widen<Tin>(reinterpret_cast<const Tin*>(slots)[i]);
        for (int s = 1; s < nslots; ++s)
            acc = combine<OP, A>(acc, widen<Tin>(reinterpret_cast<const Tin*>(slots + s * slot_stride)[i]));
        if (do_scale)
            acc = static_cast<A>(acc * static_cast<A>(scale));
        reinterpret_cast<Tout*>(out)[i] = narrow<Tout, A>(acc);
    }
}

// ------------------------------------------------------------------ reduce family
template <typename Tin, typename Tout>
__global__ void __launch_bounds__(512) reduce_family_kernel(const ReduceArgs a) {
    const CommonArgs& c = a.c;
    const int n = c.nranks, rank = c.rank;
    constexpr uint64_t V = 16 / sizeof(Tin);
    const uint64_t esz_in = sizeof(Tin), esz_out = sizeof(Tout);
    char* const my_heap = c.peers.heap[rank];
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    uint32_t epoch = c.epoch;

    if (a.one_shot) {
        // every rank pushes its whole input into slot [rank] of every peer
        const uint64_t slot_stride = round_up_u64(a.len * esz_in, 16);
        const uint64_t per_cta = round_up_u64((a.len + gridDim.x - 1) / gridDim.x, V);
        const uint64_t b = min(a.len, per_cta * blockIdx.x), e = min(a.len, b + per_cta);
        for (int jj = 0; jj < n; ++jj) {
            const int j = (rank + jj) % n;
            cta_copy(c.peers.heap[j] + a.stage_off + rank * slot_stride + b * esz_in, in + b * esz_in,
                     (e - b) * esz_in);
        }
        if (!cta_barrier(c, ++epoch))
            return;
        char* red = my_heap + a.red_off + b * esz_out;
        const char* slots = my_heap + a.stage_off + b * esz_in;
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_SUM>(slots, slot_stride, n, red, e - b, a.scale);
                break;
            case MegRay::MEGRAY_MAX:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MAX>(slots, slot_stride, n, red, e - b, a.scale);
                break;
            default:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MIN>(slots, slot_stride, n, red, e - b, a.scale);
        }
        __syncthreads();
        if (out != nullptr)
            cta_copy(out + b * esz_out, red, (e - b) * esz_out);
        return;
    }

    const uint64_t se = a.slice_elems;
    const uint64_t slot_stride = round_up_u64(se * esz_in, 16);
    const uint64_t per_cta = round_up_u64((se + gridDim.x - 1) / gridDim.x, V);
    const uint64_t sub_b = min(se, per_cta * blockIdx.x);  // this CTA's range inside every slice
    // slice j covers elements [j*se, min(len, (j+1)*se)) of the logical buffer
    auto slice_len = [&](int j) -> uint64_t {
        const uint64_t s0 = static_cast<uint64_t>(j) * se;
        return s0 >= a.len ? 0 : min(se, a.len - s0);
    };
    auto sub_range = [&](int j, uint64_t* b, uint64_t* e) {
        const uint64_t L = slice_len(j);
        *b = min(L, sub_b);
        *e = min(L, sub_b + per_cta);
    };

    // phase P: slice j of my input -> peer j's slot [rank]
    for (int jj = 0; jj < n; ++jj) {
        const int j = (rank + 1 + jj) % n;
        uint64_t b, e;
        sub_range(j, &b, &e);
        cta_copy(c.peers.heap[j] + a.stage_off + rank * slot_stride + b * esz_in,
                 in + (static_cast<uint64_t>(j) * a.in_pitch_elems + b) * esz_in, (e - b) * esz_in);
    }
    if (!cta_barrier(c, ++epoch))
        return;

    // phase R: combine the n slots of my slice, in rank order
    uint64_t b, e;
    sub_range(rank, &b, &e);
    char* red = my_heap + a.red_off + b * esz_out;
    {
        const char* slots = my_heap + a.stage_off + b * esz_in;
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_SUM>(slots, slot_stride, n, red, e - b, a.scale);
                break;
            case MegRay::MEGRAY_MAX:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MAX>(slots, slot_stride, n, red, e - b, a.scale);
                break;
            default:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MIN>(slots, slot_stride, n, red, e - b, a.scale);
        }
    }
    if (a.out_is_slice) {  // reduce_scatter: done after a local copy
        __syncthreads();
        if (out != nullptr)
            cta_copy(out + b * esz_out, red, (e - b) * esz_out);
        return;
    }
    if (!cta_barrier(c, ++epoch))
        return;

    // phase G: reduced slices from every rank's `red` into my output
    if (a.do_gather && out != nullptr) {
        for (int qq = 0; qq < n; ++qq) {
            const int q = (rank + qq) % n;
            uint64_t qb, qe;
            sub_range(q, &qb, &qe);
            cta_copy(out + (static_cast<uint64_t>(q) * se + qb) * esz_out,
                     c.peers.heap[q] + a.red_off + qb * esz_out, (qe - qb) * esz_out);
        }
    }
}

// ------------------------------------------------------------------ exchange family
__global__ void __launch_bounds__(512) exchange_family_kernel(const ExchangeArgs a) {
    const CommonArgs& c = a.c;
    const int n = c.nranks, rank = c.rank;
    char* const my_heap = c.peers.heap[rank];
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    const uint64_t chunk_stride = round_up_u64(a.chunk_bytes, 16);
    const uint64_t per_cta = round_up_u64((a.chunk_bytes + gridDim.x - 1) / gridDim.x, 16);
    const uint64_t sub_b = per_cta * blockIdx.x;
    auto sub_range = [&](uint64_t L, uint64_t* b, uint64_t* e) {
        *b = min(L, sub_b);
        *e = min(L, sub_b + per_cta);
    };
    uint32_t epoch = c.epoch;

    if (a.push_all) {
        uint64_t b, e;
        sub_range(a.chunk_bytes, &b, &e);
        for (int jj = 0; jj < n; ++jj) {
            const int j = (rank + 1 + jj) % n;
            cta_copy(c.peers.heap[j] + a.pub_off + rank * chunk_stride + b,
                     in + static_cast<uint64_t>(a.push_chunk[j]) * a.in_pitch + b, e - b);
        }
        if (!cta_barrier(c, ++epoch))
            return;
        for (int q = 0; q < n; ++q)
            cta_copy(out + static_cast<uint64_t>(q) * a.out_pitch + b, my_heap + a.pub_off + q * chunk_stride + b,
                     e - b);
        return;
    }
    // phase P
    if (a.push_root == rank) {
        // bandwidth-optimal broadcast, step 1: slice j of the message -> peer j's pub buffer
        for (int jj = 0; jj < n; ++jj) {
            const int j = (rank + 1 + jj) % n;
            uint64_t b, e;
            sub_range(a.pull_bytes[j], &b, &e);
            cta_copy(c.peers.heap[j] + a.pub_off + b, in + static_cast<uint64_t>(j) * a.in_pitch + b,
                     e - b);
        }
    } else if (a.push_root < 0) {
        uint64_t b, e;
        sub_range(a.chunk_bytes, &b, &e);
        for (int k = 0; k < a.publish_chunks; ++k)
            cta_copy(my_heap + a.pub_off + k * chunk_stride + b,
                     in + static_cast<uint64_t>(k) * a.in_pitch + b, e - b);
    }
    if (!cta_barrier(c, ++epoch))
        return;

    // phase G
    if (out == nullptr)
        return;
    for (int qq = 0; qq < n; ++qq) {
        const int q = (rank + qq) % n;
        if (!((a.pull_mask >> q) & 1u))
            continue;
        uint64_t b, e;
        sub_range(a.pull_bytes[q], &b, &e);
        cta_copy(out + static_cast<uint64_t>(a.dst_chunk[q]) * a.out_pitch + b,
                 c.peers.heap[q] + a.pub_off + static_cast<uint64_t>(a.src_chunk[q]) * chunk_stride + b,
                 e - b);
    }
}


// ------------------------------------------------------------------ direct family
// multimem (NVLS) loads: the switch combines the 16 bytes at the same heap offset of all ranks.
template <typename T, int OP>
__device__ __forceinline__ uint4 mc_ld_reduce(const void* p);

#define MC_LD(T, OP, STR)                                                                       \
    template <>                                                                                 \
    __device__ __forceinline__ uint4 mc_ld_reduce<T, OP>(const void* p) {                       \
        uint4 v;                                                                                \
        asm volatile("multimem.ld_reduce.relaxed.sys.global." STR " {%0, %1, %2, %3}, [%4];"    \
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)                               \
                     : "l"(p)                                                                   \
                     : "memory");                                                               \
        return v;                                                                               \
    }
MC_LD(__nv_bfloat16, MegRay::MEGRAY_SUM, "add.acc::f32.v4.bf16x2")
MC_LD(__nv_bfloat16, MegRay::MEGRAY_MAX, "max.v4.bf16x2")
MC_LD(__nv_bfloat16, MegRay::MEGRAY_MIN, "min.v4.bf16x2")
MC_LD(__half, MegRay::MEGRAY_SUM, "add.acc::f32.v4.f16x2")
MC_LD(__half, MegRay::MEGRAY_MAX, "max.v4.f16x2")
MC_LD(__half, MegRay::MEGRAY_MIN, "min.v4.f16x2")
MC_LD(float, MegRay::MEGRAY_SUM, "add.v4.f32")
#undef MC_LD
// combinations the switch cannot reduce are never launched with NVLS; keep the template whole
template <typename T, int OP>
__device__ __forceinline__ uint4 mc_ld_reduce(const void* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}

__device__ __forceinline__ void mc_st_v4(void* p, const uint4& v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y),
                 "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void mc_st_v2(void* p, const uint2& v) {
    asm volatile("multimem.st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y) : "memory");
}

// Reduce elements [b, e) of slice `rank`: load from all inputs, combine in rank order, scale,
// cast; store into every rank's output (all_reduce) or into `out_local` (reduce_scatter).
template <typename Tin, typename Tout, int OP, bool NVLS>
__device__ __forceinline__ void direct_reduce_range(const DirectArgs& a, uint64_t elem0, uint64_t b, uint64_t e) {
    using A = typename Acc<Tin>::type;
    constexpr int V = 16 / sizeof(Tin);
    constexpr int OB = V * sizeof(Tout);
    const int n = a.c.nranks;
    const bool do_scale = IsFloatAcc<A>::value && OP == MegRay::MEGRAY_SUM && a.scale != 1.0f;
    const bool to_all = a.kind == DIRECT_ALL_REDUCE;
    const uint64_t nvec = (e - b) / V;
    // byte positions relative to the start of every rank's input / output buffer
    const uint64_t in_byte0 = (elem0 + b) * sizeof(Tin);
    // all_reduce writes the slice back at the same element positions; reduce_scatter writes the
    // slice to the start of the local result
    const uint64_t out_byte0 = to_all ? (elem0 + b) * sizeof(Tout) : b * sizeof(Tout);
    // U independent vectors per thread and iteration: all their loads are issued before the
    // first use, which is what keeps enough bytes in flight to fill the links
    constexpr int U = NVLS ? 4 : 2;
    for (uint64_t i0 = threadIdx.x; i0 < nvec; i0 += static_cast<uint64_t>(U) * blockDim.x) {
        A acc[U][V];
        if (NVLS) {
            uint4 raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
                if (i < nvec)
                    raw[u] = mc_ld_reduce<Tin, OP>(a.mc_base + a.in_off + in_byte0 + i * 16);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const Tin* el = reinterpret_cast<const Tin*>(&raw[u]);
#pragma unroll
                for (int k = 0; k < V; ++k)
                    acc[u][k] = widen<Tin>(el[k]);
            }
        } else {
            uint4 raw[U][kMaxRanks];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
#pragma unroll
                for (int q = 0; q < kMaxRanks; ++q)
                    if (q < n && i < nvec)
                        raw[u][q] = ld_cg_v4(a.in_base[q] + in_byte0 + i * 16);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int q = 0; q < kMaxRanks; ++q) {
                    if (q < n) {
                        const Tin* el = reinterpret_cast<const Tin*>(&raw[u][q]);
#pragma unroll
                        for (int k = 0; k < V; ++k)
                            acc[u][k] = q == 0 ? widen<Tin>(el[k]) : combine<OP, A>(acc[u][k], widen<Tin>(el[k]));
                    }
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
            if (i >= nvec)
                break;
            Tout o[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                if (do_scale)
                    acc[u][k] = static_cast<A>(acc[u][k] * static_cast<A>(a.scale));
                o[k] = narrow<Tout, A>(acc[u][k]);
            }
            if (!to_all) {
                char* dst = static_cast<char*>(a.out_local) + out_byte0 + i * OB;
                if (OB >= 16) {
#pragma unroll
                    for (int w = 0; w < OB / 16; ++w)
                        reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(o)[w];
                } else {
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
                }
            } else if (NVLS) {
                char* dst = a.mc_base + a.out_off + out_byte0 + i * OB;
                if (OB >= 16) {
#pragma unroll
                    for (int w = 0; w < OB / 16; ++w)
                        mc_st_v4(dst + 16 * w, reinterpret_cast<const uint4*>(o)[w]);
                } else {
                    mc_st_v2(dst, *reinterpret_cast<const uint2*>(o));
                }
            } else {
#pragma unroll
                for (int q = 0; q < kMaxRanks; ++q) {
                    if (q < n) {
                        char* dst = a.out_base[(a.c.rank + q) % n] + out_byte0 + i * OB;
                        if (OB >= 16) {
#pragma unroll
                            for (int w = 0; w < OB / 16; ++w)
                                reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(o)[w];
                        } else {
                            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
                        }
                    }
                }
            }
        }
    }
    // element tail (fewer than V elements): plain peer accesses
    for (uint64_t i = b + nvec * V + threadIdx.x; i < e; i += blockDim.x) {
        A acc = widen<Tin>(reinterpret_cast<const Tin*>(a.in_base[0])[elem0 + i]);
        for (int q = 1; q < n; ++q)
            acc = combine<OP, A>(acc, widen<Tin>(reinterpret_cast<const Tin*>(a.in_base[q])[elem0 + i]));
        if (do_scale)
            acc = static_cast<A>(acc * static_cast<A>(a.scale));
        const Tout o = narrow<Tout, A>(acc);
        if (!to_all) {
            static_cast<Tout*>(a.out_local)[i] = o;
        } else {
            for (int q = 0; q < n; ++q)
                reinterpret_cast<Tout*>(a.out_base[q])[elem0 + i] = o;
        }
    }
}

template <typename Tin, typename Tout, bool NVLS>
__global__ void __launch_bounds__(512) direct_family_kernel(const DirectArgs a) {
    const CommonArgs& c = a.c;
    const int n = c.nranks, rank = c.rank;
    constexpr uint64_t V = 16 / sizeof(Tin);
    uint32_t epoch = c.epoch;
    // inputs are final / outputs may be overwritten on every rank
    if (!cta_barrier(c, ++epoch))
        return;
    if (a.kind == DIRECT_ALL_GATHER) {
        // this rank's block into slot `rank` of every output
        const uint64_t bytes = a.len * sizeof(Tin);
        const uint64_t per_cta = round_up_u64((bytes + gridDim.x - 1) / gridDim.x, 16);
        const uint64_t b = min(bytes, per_cta * blockIdx.x), e = min(bytes, b + per_cta);
        const char* src = static_cast<const char*>(a.in_local);
        if (NVLS && ((reinterpret_cast<uintptr_t>(src) | (a.out_off + rank * bytes)) & 15) == 0) {  // (heap-resident output)
            char* dst = a.mc_base + a.out_off + rank * bytes;
            const uint64_t nv = (e - b) / 16;
            for (uint64_t i = threadIdx.x; i < nv; i += blockDim.x)
                mc_st_v4(dst + b + i * 16, ld_cg_v4(src + b + i * 16));
            for (uint64_t k = b + nv * 16 + threadIdx.x; k < e; k += blockDim.x)
                for (int q = 0; q < n; ++q)
                    (a.out_base[q] + rank * bytes)[k] = src[k];
        } else {
            for (int qq = 0; qq < n; ++qq) {
                const int q = (rank + qq) % n;
                cta_copy(a.out_base[q] + rank * bytes + b, src + b, e - b);
            }
        }
    } else if (a.kind == DIRECT_ALL_TO_ALL) {
        // chunk q of the input into slot `rank` of rank q's output, starting with rank+1
        const uint64_t bytes = a.len * sizeof(Tin);
        const uint64_t per_cta = round_up_u64((bytes + gridDim.x - 1) / gridDim.x, 16);
        const uint64_t b = min(bytes, per_cta * blockIdx.x), e = min(bytes, b + per_cta);
        const char* src = static_cast<const char*>(a.in_local);
        for (int qq = 1; qq <= n; ++qq) {
            const int q = (rank + qq) % n;
            cta_copy(a.out_base[q] + rank * bytes + b, src + q * bytes + b, e - b);
        }
    } else {
        // slice `rank`: all_reduce splits len into n slices of se elements, reduce_scatter's
        // slice is the rank-th block of len elements
        uint64_t se, elem0, L;
        if (a.kind == DIRECT_ALL_REDUCE) {
            se = round_up_u64((a.len + n - 1) / n, V);
            elem0 = min(a.len, se * rank);
            L = min(a.len, elem0 + se) - elem0;
        } else {
            elem0 = a.len * rank;
            L = a.len;
        }
        const uint64_t per_cta = round_up_u64((L + gridDim.x - 1) / gridDim.x, V);
        const uint64_t b = min(L, per_cta * blockIdx.x), e = min(L, b + per_cta);
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_SUM, NVLS>(a, elem0, b, e);
                break;
            case MegRay::MEGRAY_MAX:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MAX, NVLS>(a, elem0, b, e);
                break;
            default:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MIN, NVLS>(a, elem0, b, e);
        }
    }
    // all transfers are complete before any rank uses its output or overwrites its input
    cta_barrier(c, ++epoch);
}

// ------------------------------------------------------------------ stand-alone reduce_n
struct ReduceNArgs {
    const void* in[kMaxRanks];
    void* out;
    uint64_t len;
    float scale;
    int n_in;
    int op;
};

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(512) reduce_n_kernel(const ReduceNArgs a) {
    using A = typename Acc<Tin>::type;
    constexpr int V = 16 / sizeof(Tin);
    const uint64_t nvec = a.len / V;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const uint64_t gid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    bool aligned = (reinterpret_cast<uintptr_t>(a.out) & 15) == 0;
    for (int s = 0; s < a.n_in; ++s)
        aligned = aligned && (reinterpret_cast<uintptr_t>(a.in[s]) & 15) == 0;
    const bool do_scale = IsFloatAcc<A>::value && a.op == MegRay::MEGRAY_SUM && a.scale != 1.0f;
    auto comb = [&](A x, A y) -> A {
        if (a.op == MegRay::MEGRAY_SUM)
            return static_cast<A>(x + y);
        if (a.op == MegRay::MEGRAY_MAX)
            return x > y ? x : y;
        return x < y ? x : y;
    };
    uint64_t first_scalar = 0;
    if (aligned) {
        first_scalar = nvec * V;
        for (uint64_t i = gid; i < nvec; i += stride) {
            A acc[V];
            // all inputs' loads are issued before the first use
            uint4 raw[kMaxRanks];
#pragma unroll
            for (int s = 0; s < kMaxRanks; ++s)
                if (s < a.n_in)
                    raw[s] = ld_cg_v4(static_cast<const char*>(a.in[s]) + i * 16);
            {
                const Tin* e = reinterpret_cast<const Tin*>(&raw[0]);
#pragma unroll
                for (int k = 0; k < V; ++k)
                    acc[k] = widen<Tin>(e[k]);
            }
#pragma unroll
            for (int s = 1; s < kMaxRanks; ++s) {
                if (s < a.n_in) {
                    const Tin* e = reinterpret_cast<const Tin*>(&raw[s]);
#pragma unroll
                    for (int k = 0; k < V; ++k)
                        acc[k] = comb(acc[k], widen<Tin>(e[k]));
                }
            }
            Tout o[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                if (do_scale)
                    acc[k] = static_cast<A>(acc[k] * static_cast<A>(a.scale));
                o[k] = narrow<Tout, A>(acc[k]);
            }
            constexpr int OB = V * sizeof(Tout);
            char* dst = static_cast<char*>(a.out) + i * OB;
            if (OB >= 16) {
#pragma unroll
                for (int b = 0; b < OB / 16; ++b)
                    reinterpret_cast<uint4*>(dst)[b] = reinterpret_cast<const uint4*>(o)[b];
            } else {
                *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
            }
        }
    }
    for (uint64_t i = first_scalar + gid; i < a.len; i += stride) {
        A acc = widen<Tin>(static_cast<const Tin*>(a.in[0])[i]);
        for (int s = 1; s < a.n_in; ++s)
            acc = comb(acc, widen<Tin>(static_cast<const Tin*>(a.in[s])[i]));
        if (do_scale)
            acc = static_cast<A>(acc * static_cast<A>(a.scale));
        static_cast<Tout*>(a.out)[i] = narrow<Tout, A>(acc);
    }
}

// ------------------------------------------------------------------ dispatch
template <typename Tin, typename Tout>
cudaError_t run_reduce(const ReduceArgs& a, int ctas, int threads, cudaStream_t s) {
    reduce_family_kernel<Tin, Tout><<<ctas, threads, 0, s>>>(a);
    count_launch();
    return cudaGetLastError();
}
template <typename Tin, typename Tout>
cudaError_t run_reduce_n(const ReduceNArgs& a, cudaStream_t s) {
    constexpr int V = 16 / sizeof(Tin);
    uint64_t vecs = a.len / V + 1;
    int threads = 256;
    uint64_t blocks = (vecs + threads - 1) / threads;
    if (blocks > 148 * 8)
        blocks = 148 * 8;
    reduce_n_kernel<Tin, Tout><<<static_cast<int>(blocks), threads, 0, s>>>(a);
    count_launch();
    return cudaGetLastError();
}

// Calls f.template operator()<Tin, Tout>() for the supported (in, out) dtype pairs:
// equal dtypes for all ten numeric types, and any pair of {fp16, bf16, fp32}.
template <typename F>
cudaError_t dispatch_types(DType in, DType out, F&& f) {
    using namespace MegRay;
    if (in == out) {
        switch (in) {
            case MEGRAY_INT8: return f.template operator()<int8_t, int8_t>();
            case MEGRAY_UINT8: return f.template operator()<uint8_t, uint8_t>();
            case MEGRAY_INT32: return f.template operator()<int32_t, int32_t>();
            case MEGRAY_UINT32: return f.template operator()<uint32_t, uint32_t>();
            case MEGRAY_INT64: return f.template operator()<int64_t, int64_t>();
            case MEGRAY_UINT64: return f.template operator()<uint64_t, uint64_t>();
            case MEGRAY_FLOAT16: return f.template operator()<__half, __half>();
            case MEGRAY_BFLOAT16: return f.template operator()<__nv_bfloat16, __nv_bfloat16>();
            case MEGRAY_FLOAT32: return f.template operator()<float, float>();
            case MEGRAY_FLOAT64: return f.template operator()<double, double>();
            default: return cudaErrorInvalidValue;
        }
    }
    if (in == MEGRAY_FLOAT32 && out == MEGRAY_BFLOAT16) return f.template operator()<float, __nv_bfloat16>();
    if (in == MEGRAY_FLOAT32 && out == MEGRAY_FLOAT16) return f.template operator()<float, __half>();
    if (in == MEGRAY_BFLOAT16 && out == MEGRAY_FLOAT32) return f.template operator()<__nv_bfloat16, float>();
    if (in == MEGRAY_FLOAT16 && out == MEGRAY_FLOAT32) return f.template operator()<__half, float>();
    if (in == MEGRAY_BFLOAT16 && out == MEGRAY_FLOAT16) return f.template operator()<__nv_bfloat16, __half>();
    if (in == MEGRAY_FLOAT16 && out == MEGRAY_BFLOAT16) return f.template operator()<__half, __nv_bfloat16>();
    return cudaErrorInvalidValue;
}

struct ReduceLauncher {
    const ReduceArgs& a;
    int ctas, threads;
    cudaStream_t s;
    template <typename Tin, typename Tout>
    cudaError_t operator()() const {
        return run_reduce<Tin, Tout>(a, ctas, threads, s);
    }
};
struct DirectLauncher {
    const DirectArgs& a;
    int ctas, threads;
    cudaStream_t s;
    template <typename Tin, typename Tout>
    cudaError_t operator()() const {
        if (a.mc_base != nullptr)
            direct_family_kernel<Tin, Tout, true><<<ctas, threads, 0, s>>>(a);
        else
            direct_family_kernel<Tin, Tout, false><<<ctas, threads, 0, s>>>(a);
        count_launch();
        return cudaGetLastError();
    }
};
struct ReduceNLauncher {
    const ReduceNArgs& a;
    cudaStream_t s;
    template <typename Tin, typename Tout>
    cudaError_t operator()() const {
        return run_reduce_n<Tin, Tout>(a, s);
    }
};

}  // namespace

cudaError_t launch_reduce(const ReduceArgs& a, int ctas, int threads, cudaStream_t stream) {
    if (ctas < 1 || ctas > kMaxCtas || threads < 32 || threads > 512 || a.c.nranks < 1 ||
        a.c.nranks > kMaxRanks)
        return cudaErrorInvalidValue;
    return dispatch_types(a.in_dtype, a.out_dtype, ReduceLauncher{a, ctas, threads, stream});
}

bool nvls_supports(DType in_dtype, DType out_dtype, ReduceOp op) {
    using namespace MegRay;
    if (in_dtype == MEGRAY_BFLOAT16 || in_dtype == MEGRAY_FLOAT16)
        return out_dtype == in_dtype || out_dtype == MEGRAY_FLOAT32 || out_dtype == MEGRAY_BFLOAT16 ||
               out_dtype == MEGRAY_FLOAT16;
    if (in_dtype == MEGRAY_FLOAT32)
        return op == MEGRAY_SUM &&
               (out_dtype == MEGRAY_FLOAT32 || out_dtype == MEGRAY_BFLOAT16 || out_dtype == MEGRAY_FLOAT16);
    return false;
}

cudaError_t launch_direct(const DirectArgs& a, int ctas, int threads, cudaStream_t stream) {
    if (ctas < 1 || ctas > kMaxCtas || threads < 32 || threads > 512 || a.c.nranks < 1 ||
        a.c.nranks > kMaxRanks)
        return cudaErrorInvalidValue;
    if (a.mc_base != nullptr && (a.kind == DIRECT_ALL_REDUCE || a.kind == DIRECT_REDUCE_SCATTER) &&
        !nvls_supports(a.in_dtype, a.out_dtype, a.op))
        return cudaErrorInvalidValue;
    return dispatch_types(a.in_dtype, a.out_dtype, DirectLauncher{a, ctas, threads, stream});
}

cudaError_t launch_exchange(const ExchangeArgs& a, int ctas, int threads, cudaStream_t stream) {
    if (ctas < 1 || ctas > kMaxCtas || threads < 32 || threads > 512 || a.c.nranks < 1 ||
        a.c.nranks > kMaxRanks)
        return cudaErrorInvalidValue;
    exchange_family_kernel<<<ctas, threads, 0, stream>>>(a);
    count_launch();
    return cudaGetLastError();
}

cudaError_t launch_reduce_n(const void* const* in, int n_in, void* out, uint64_t len, DType in_dtype,
                            DType out_dtype, ReduceOp op, float scale, cudaStream_t stream) {
    if (n_in < 1 || n_in > kMaxRanks)
        return cudaErrorInvalidValue;
    if (len == 0)
        return cudaSuccess;
    ReduceNArgs a;
    for (int i = 0; i < kMaxRanks; ++i)
        a.in[i] = i < n_in ? in[i] : nullptr;
    a.out = out;
    a.len = len;
    a.scale = scale;
    a.n_in = n_in;
    a.op = op;
    return dispatch_types(in_dtype, out_dtype, ReduceNLauncher{a, stream});
}

}  // namespace coll
}  // namespace mgk
