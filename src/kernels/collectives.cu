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

// ------------------------------------------------------------------ phase stamps
__device__ __forceinline__ void stamp(const CommonArgs& c, int i) {
    if (c.phases && blockIdx.x == 0 && threadIdx.x == 0 && i < kMaxPhases)
        reinterpret_cast<uint64_t*>(c.peers.heap[c.rank] + kPhaseOff)[i] = globaltimer_ns();
}

// ------------------------------------------------------------------ failure record
// The first wait that runs out (or lookup that fails) sets the status word and leaves, in the
// pad at kDebugOff + 32, what it was: {source line, detail (peer, entry, target, ...), rank}.
__device__ __forceinline__ void fail_with(const CommonArgs& c, int code, int line, uint64_t detail) {
    if (c.status != nullptr && atomicCAS(c.status, 0, code) == 0) {
        uint64_t* rec = reinterpret_cast<uint64_t*>(c.peers.heap[c.rank] + kDebugOff + 32);
        rec[0] = static_cast<uint64_t>(static_cast<uint32_t>(line));
        rec[1] = detail;
        rec[2] = static_cast<uint64_t>(c.rank);
    }
}
#define FAIL_WITH(c, code, detail) fail_with((c), (code), __LINE__, (detail))

// ------------------------------------------------------------------ range guard
// In a build with MEGRAY_DEBUG_BOUNDS every CTA-level primitive asks the guard before it touches
// a range.  Allowed: any rank's heap, this call's local buffers, and (single-pass kernels on
// exchanged addresses) the peers' buffers.  In an ordinary build the guard is empty and free.
struct Guard {
#ifdef MEGRAY_DEBUG_BOUNDS
    const CommonArgs* c;
    const char* peer_in[kMaxRanks];
    const char* peer_out[kMaxRanks];
    __device__ __forceinline__ bool inside(const char* p, uint64_t n, const char* lo, uint64_t len) const {
        return lo != nullptr && len != 0 && p >= lo && p + n <= lo + len;
    }
    __device__ bool ok(const void* ptr, uint64_t n, int line) const {
        if (n == 0)
            return true;
        const char* p = static_cast<const char*>(ptr);
        bool fine = inside(p, n, static_cast<const char*>(c->guard_in), c->guard_in_bytes) ||
                    inside(p, n, static_cast<const char*>(c->guard_out), c->guard_out_bytes);
        for (int q = 0; q < c->nranks && !fine; ++q)
            fine = inside(p, n, c->peers.heap[q], c->heap_bytes) ||
                   inside(p, n, peer_in[q], c->guard_peer_in_bytes) ||
                   inside(p, n, peer_out[q], c->guard_peer_out_bytes);
        if (!fine && c->status != nullptr && atomicCAS(c->status, 0, kStatusOutOfBounds) == 0) {
            uint64_t* rec = reinterpret_cast<uint64_t*>(c->peers.heap[c->rank] + kDebugOff);
            rec[0] = reinterpret_cast<uint64_t>(ptr);
            rec[1] = n;
            rec[2] = static_cast<uint64_t>(static_cast<uint32_t>(line)) | (static_cast<uint64_t>(c->rank) << 32);
        }
        return fine;
    }
#else
    __device__ __forceinline__ bool ok(const void*, uint64_t, int) const { return true; }
#endif
};
__device__ __forceinline__ Guard make_guard(const CommonArgs& c) {
    Guard g;
#ifdef MEGRAY_DEBUG_BOUNDS
    g.c = &c;
    for (int q = 0; q < kMaxRanks; ++q)
        g.peer_in[q] = g.peer_out[q] = nullptr;
#endif
    return g;
}
#define GUARD_OK(g, p, n) (g).ok((p), (n), __LINE__)

// ------------------------------------------------------------------ waits
// A wait that has lasted a while pauses between polls (when spin_sleep_ns is set): a rank that
// waits for long, such as the root of a reduce or CTAs that finished early, then keeps its L2
// free for the peers that read and write this GPU's memory.  The first polls go back to back,
// which is all that ranks running in step ever need.
__device__ __forceinline__ void poll_backoff(const CommonArgs& c, uint32_t spins) {
    if (c.spin_sleep_ns != 0 && spins > 32)
        __nanosleep(c.spin_sleep_ns);
}

// Wait until *flag has reached `target` (wrap-safe).  False when the wait ran out, in which case
// the status word says so.
// `what` goes into the failure record: 1 barrier, 2 chunk announcement, 3 consumed-chunk counter.
__device__ __forceinline__ bool wait_flag_reached(const CommonArgs& c, const uint32_t* flag, uint32_t target, int what = 1) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flag) - target) < 0) {
        if ((++spins & 63) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > c.timeout_ns) {
                FAIL_WITH(c, kStatusTimeout, (static_cast<uint64_t>(what) << 32) | target);
                return false;
            }
        }
        poll_backoff(c, spins);
    }
    return true;
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
        ok = wait_flag_reached(c, mine, target) ? 1 : 0;
    }
    return __syncthreads_and(ok) != 0;
}

// ------------------------------------------------------------------ copies
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
    return __ldcg(reinterpret_cast<const uint4*>(p));
}
// (a peer GPU may have written the byte: read it where its store landed, in L2)
__device__ __forceinline__ char ld_cg_byte(const char* p) {
    return static_cast<char>(__ldcg(reinterpret_cast<const unsigned char*>(p)));
}

// CTA-cooperative byte copy for any alignment.  Vector (16 B) body when source and
// destination are equally aligned, else 4-byte or 1-byte units.
// `tid` of `nth` threads take part (the whole CTA in cta_copy below).
__device__ __forceinline__ void cta_copy_part(const Guard& g, char* dst, const char* src, uint64_t nbytes,
                                              unsigned tid, unsigned nth) {
    if (nbytes == 0)
        return;
    if (!GUARD_OK(g, dst, nbytes) || !GUARD_OK(g, src, nbytes))
        return;
    const uintptr_t da = reinterpret_cast<uintptr_t>(dst), sa = reinterpret_cast<uintptr_t>(src);
    if (((da ^ sa) & 15) == 0) {
        uint64_t head = (16 - (da & 15)) & 15;
        if (head > nbytes)
            head = nbytes;
        for (uint64_t i = tid; i < head; i += nth)
            dst[i] = ld_cg_byte(src + i);
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
            dst[k] = ld_cg_byte(src + k);
    } else if (((da | sa | nbytes) & 3) == 0) {
        const uint32_t* s = reinterpret_cast<const uint32_t*>(src);
        uint32_t* d = reinterpret_cast<uint32_t*>(dst);
        for (uint64_t i = tid; i < nbytes / 4; i += nth)
            d[i] = __ldcg(s + i);
    } else {
        for (uint64_t i = tid; i < nbytes; i += nth)
            dst[i] = ld_cg_byte(src + i);
    }
}

__device__ __forceinline__ void cta_copy(const Guard& g, char* dst, const char* src, uint64_t nbytes) {
    cta_copy_part(g, dst, src, nbytes, threadIdx.x, blockDim.x);
}

// Named barriers (ids 1..15; id 0 is __syncthreads): `count` threads in all, some of which only
// arrive and go on, while the others wait for them.
__device__ __forceinline__ void named_bar_arrive(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// Progress of the storing warps of a root CTA, for its announcing warp.  A warp that has issued
// all its stores of round k - 1 writes k into its word (release at CTA scope, after the warp has
// converged); the announcing warp reads all words (acquire) and takes the minimum.  Its releasing
// store at system scope then also covers the storing warps' stores.
__device__ __forceinline__ void warp_round_done(uint32_t* s_round, uint32_t rounds) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) {
        __threadfence_block();
        reinterpret_cast<volatile uint32_t*>(s_round)[threadIdx.x >> 5] = rounds;
    }
}
__device__ __forceinline__ uint32_t rounds_done_by_all(const uint32_t* s_round, unsigned warps) {
    const unsigned lane = threadIdx.x & 31;
    uint32_t m = lane < warps ? reinterpret_cast<const volatile uint32_t*>(s_round)[lane] : 0xffffffffu;
    m = __reduce_min_sync(0xffffffffu, m);
    __threadfence_block();
    return m;
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
__device__ __forceinline__ void cta_reduce_slots(const Guard& g, const char* slots, uint64_t slot_stride,
                                                 int nslots, char* out, uint64_t n, float scale) {
    using A = typename Acc<Tin>::type;
    if (n == 0 || !GUARD_OK(g, out, n * sizeof(Tout)) ||
        !GUARD_OK(g, slots, (nslots - 1) * slot_stride + n * sizeof(Tin)))
        return;
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
    const Guard g = make_guard(c);
    stamp(c, 0);
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
            cta_copy(g, c.peers.heap[j] + a.stage_off + rank * slot_stride + b * esz_in, in + b * esz_in,
                     (e - b) * esz_in);
        }
        if (!cta_barrier(c, ++epoch))
            return;
        char* red = my_heap + a.red_off + b * esz_out;
        const char* slots = my_heap + a.stage_off + b * esz_in;
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_SUM>(g, slots, slot_stride, n, red, e - b, a.scale);
                break;
            case MegRay::MEGRAY_MAX:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MAX>(g, slots, slot_stride, n, red, e - b, a.scale);
                break;
            default:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MIN>(g, slots, slot_stride, n, red, e - b, a.scale);
        }
        __syncthreads();
        if (out != nullptr)
            cta_copy(g, out + b * esz_out, red, (e - b) * esz_out);
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
        cta_copy(g, c.peers.heap[j] + a.stage_off + rank * slot_stride + b * esz_in,
                 in + (static_cast<uint64_t>(j) * a.in_pitch_elems + b) * esz_in, (e - b) * esz_in);
    }
    stamp(c, 1);
    if (!cta_barrier(c, ++epoch))
        return;
    stamp(c, 2);

    // phase R: combine the n slots of my slice, in rank order
    uint64_t b, e;
    sub_range(rank, &b, &e);
    char* red = my_heap + a.red_off + b * esz_out;
    {
        const char* slots = my_heap + a.stage_off + b * esz_in;
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_SUM>(g, slots, slot_stride, n, red, e - b, a.scale);
                break;
            case MegRay::MEGRAY_MAX:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MAX>(g, slots, slot_stride, n, red, e - b, a.scale);
                break;
            default:
                cta_reduce_slots<Tin, Tout, MegRay::MEGRAY_MIN>(g, slots, slot_stride, n, red, e - b, a.scale);
        }
    }
    if (a.out_is_slice) {  // reduce_scatter: done after a local copy
        __syncthreads();
        if (out != nullptr)
            cta_copy(g, out + b * esz_out, red, (e - b) * esz_out);
        return;
    }
    stamp(c, 3);
    if (!cta_barrier(c, ++epoch))
        return;
    stamp(c, 4);

    // phase G: reduced slices from every rank's `red` into my output
    if (a.do_gather && out != nullptr) {
        for (int qq = 0; qq < n; ++qq) {
            const int q = (rank + qq) % n;
            uint64_t qb, qe;
            sub_range(q, &qb, &qe);
            cta_copy(g, out + (static_cast<uint64_t>(q) * se + qb) * esz_out,
                     c.peers.heap[q] + a.red_off + qb * esz_out, (qe - qb) * esz_out);
        }
    }
    stamp(c, 5);
}

// ------------------------------------------------------------------ exchange family
__global__ void __launch_bounds__(512) exchange_family_kernel(const ExchangeArgs a) {
    const CommonArgs& c = a.c;
    const Guard g = make_guard(c);
    stamp(c, 0);
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
            cta_copy(g, c.peers.heap[j] + a.pub_off + rank * chunk_stride + b,
                     in + static_cast<uint64_t>(a.push_chunk[j]) * a.in_pitch + b, e - b);
        }
        if (!cta_barrier(c, ++epoch))
            return;
        for (int q = 0; q < n; ++q)
            cta_copy(g, out + static_cast<uint64_t>(q) * a.out_pitch + b, my_heap + a.pub_off + q * chunk_stride + b,
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
            cta_copy(g, c.peers.heap[j] + a.pub_off + b, in + static_cast<uint64_t>(j) * a.in_pitch + b,
                     e - b);
        }
    } else if (a.push_root < 0) {
        uint64_t b, e;
        sub_range(a.chunk_bytes, &b, &e);
        for (int k = 0; k < a.publish_chunks; ++k)
            cta_copy(g, my_heap + a.pub_off + k * chunk_stride + b,
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
        cta_copy(g, out + static_cast<uint64_t>(a.dst_chunk[q]) * a.out_pitch + b,
                 c.peers.heap[q] + a.pub_off + static_cast<uint64_t>(a.src_chunk[q]) * chunk_stride + b,
                 e - b);
    }
}


// ------------------------------------------------------------------ small messages: flagged words
__device__ __forceinline__ void st_ll_v4(void* p, uint32_t d0, uint32_t d1, uint32_t flag) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
                 : "memory");
}
__device__ __forceinline__ uint4 ld_ll_v4(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p)
                 : "memory");
    return v;
}

// 16 bytes of payload starting at p, of which `valid` (1..16) exist; the rest reads as zero.
__device__ __forceinline__ uint4 load16_any(const char* p, uint32_t valid) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if (valid == 16 && (a & 15) == 0)
        return *reinterpret_cast<const uint4*>(p);
    uint32_t w[4] = {0u, 0u, 0u, 0u};
    if ((a & 3) == 0 && (valid & 3) == 0) {
        for (uint32_t i = 0; i < valid / 4; ++i)
            w[i] = reinterpret_cast<const uint32_t*>(p)[i];
    } else {
        for (uint32_t i = 0; i < valid; ++i)
            w[i >> 2] |= static_cast<uint32_t>(static_cast<unsigned char>(p[i])) << (8 * (i & 3));
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}
__device__ __forceinline__ void store16_any(char* p, const uint4& v, uint32_t valid) {
    const uintptr_t a = reinterpret_cast<uintptr_t>(p);
    if (valid == 16 && (a & 15) == 0) {
        *reinterpret_cast<uint4*>(p) = v;
        return;
    }
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if ((a & 3) == 0 && (valid & 3) == 0) {
        for (uint32_t i = 0; i < valid / 4; ++i)
            reinterpret_cast<uint32_t*>(p)[i] = w[i];
    } else {
        for (uint32_t i = 0; i < valid; ++i)
            p[i] = static_cast<char>(w[i >> 2] >> (8 * (i & 3)));
    }
}

// Unit u (16 bytes of payload, 32 bytes of flagged words) of a slot, once all its words carry `seq`.
// Returns false when the wait ran out.
__device__ __forceinline__ bool ll_wait_unit(const char* slot, uint64_t u, uint32_t seq, const CommonArgs& c,
                                             uint4* out) {
    const char* p = slot + u * 32;
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
        const uint4 a = ld_ll_v4(p), b = ld_ll_v4(p + 16);
        if (a.y == seq && a.w == seq && b.y == seq && b.w == seq) {
            *out = make_uint4(a.x, a.z, b.x, b.z);
            return true;
        }
        if ((++spins & 255) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > c.timeout_ns) {
                FAIL_WITH(c, kStatusTimeout, 0);
                return false;
            }
        }
    }
}

template <typename Tin, typename Tout>
__global__ void __launch_bounds__(512) ll_family_kernel(const LLArgs a) {
    using A = typename Acc<Tin>::type;
    constexpr int V = 16 / sizeof(Tin);
    const CommonArgs& c = a.c;
    const int n = c.nranks, rank = c.rank;
    const uint64_t units = (a.bytes + 15) / 16;
    const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const uint64_t gthreads = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    const char* in = static_cast<const char*>(a.in);
    char* out = static_cast<char*>(a.out);
    char* const my_slots = c.peers.heap[rank] + a.slot_off;
    const Guard g = make_guard(c);
    stamp(c, 0);
#ifdef MEGRAY_DEBUG_BOUNDS
    {
        // every range this kernel will touch, checked once: the slots it writes and reads, the
        // parts of `in` it sends and of `out` it fills
        bool fine = true;
        for (int j = 0; j < n && fine; ++j) {
            if ((a.send_mask >> j) & 1u)
                fine = GUARD_OK(g, c.peers.heap[j] + a.slot_off + static_cast<uint64_t>(rank) * kLLSlotBytes, units * 32) &&
                       GUARD_OK(g, in + a.send_off[j], a.bytes);
            if (fine && ((a.recv_mask >> j) & 1u)) {
                fine = GUARD_OK(g, my_slots + static_cast<uint64_t>(j) * kLLSlotBytes, units * 32);
                if (fine && !a.reduce && out != nullptr)
                    fine = GUARD_OK(g, out + a.recv_off[j], a.bytes);
            }
        }
        if (fine && a.self)
            fine = GUARD_OK(g, in + a.send_off[rank], a.bytes) &&
                   (out == nullptr || GUARD_OK(g, out + (a.reduce ? 0 : a.recv_off[rank]),
                                               a.reduce ? a.bytes / sizeof(Tin) * sizeof(Tout) : a.bytes));
        if (fine && a.reduce && out != nullptr)
            fine = GUARD_OK(g, out, a.bytes / sizeof(Tin) * sizeof(Tout));
        if (!fine)
            return;
    }
#endif

    // rooted operations: tell every peer that this rank has started this call
    if (a.tokens && blockIdx.x == 0 && threadIdx.x < static_cast<unsigned>(n) && static_cast<int>(threadIdx.x) != rank) {
        uint32_t* tok = reinterpret_cast<uint32_t*>(c.peers.heap[threadIdx.x] + a.token_off) + rank * 2;
        asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(tok), "r"(a.seq) : "memory");
    }
    // send: unit by unit, every destination in turn (starting with rank + 1)
    if (a.send_mask != 0) {
        for (uint64_t u = gtid; u < units; u += gthreads) {
            const uint32_t valid = static_cast<uint32_t>(min(static_cast<uint64_t>(16), a.bytes - u * 16));
            uint4 v = make_uint4(0, 0, 0, 0);
            int64_t last_off = -1;
            for (int jj = 1; jj < n; ++jj) {
                const int j = (rank + jj) % n;
                if (!((a.send_mask >> j) & 1u))
                    continue;
                if (a.send_off[j] != last_off) {  // (the same payload for every destination is read once)
                    v = load16_any(in + a.send_off[j] + u * 16, valid);
                    last_off = a.send_off[j];
                }
                char* dst = c.peers.heap[j] + a.slot_off + static_cast<uint64_t>(rank) * kLLSlotBytes + u * 32;
                st_ll_v4(dst, v.x, v.y, a.seq);
                st_ll_v4(dst + 16, v.z, v.w, a.seq);
            }
        }
    }
    stamp(c, 1);
    // receive
    bool ok = true;
    if (!a.reduce) {
        if (a.self && out != nullptr) {
            for (uint64_t u = gtid; u < units; u += gthreads) {
                const uint32_t valid = static_cast<uint32_t>(min(static_cast<uint64_t>(16), a.bytes - u * 16));
                store16_any(out + a.recv_off[rank] + u * 16, load16_any(in + a.send_off[rank] + u * 16, valid), valid);
            }
        }
        for (int qq = 1; qq < n && ok; ++qq) {
            const int q = (rank + n - qq) % n;
            if (!((a.recv_mask >> q) & 1u))
                continue;
            const char* slot = my_slots + static_cast<uint64_t>(q) * kLLSlotBytes;
            for (uint64_t u = gtid; u < units; u += gthreads) {
                uint4 v;
                if (!ll_wait_unit(slot, u, a.seq, c, &v)) {
                    ok = false;
                    break;
                }
                const uint32_t valid = static_cast<uint32_t>(min(static_cast<uint64_t>(16), a.bytes - u * 16));
                store16_any(out + a.recv_off[q] + u * 16, v, valid);
            }
        }
    } else if ((a.recv_mask != 0 || a.self) && out != nullptr) {
        const bool do_scale = IsFloatAcc<A>::value && a.op == MegRay::MEGRAY_SUM && a.scale != 1.0f;
        for (uint64_t u = gtid; u < units && ok; u += gthreads) {
            const uint32_t valid = static_cast<uint32_t>(min(static_cast<uint64_t>(16), a.bytes - u * 16));
            A acc[V];
            bool first = true;
            for (int q = 0; q < n; ++q) {
                uint4 raw;
                if (q == rank) {
                    if (!a.self)
                        continue;
                    raw = load16_any(in + a.send_off[rank] + u * 16, valid);
                } else {
                    if (!((a.recv_mask >> q) & 1u))
                        continue;
                    if (!ll_wait_unit(my_slots + static_cast<uint64_t>(q) * kLLSlotBytes, u, a.seq, c, &raw)) {
                        ok = false;
                        break;
                    }
                }
                const Tin* el = reinterpret_cast<const Tin*>(&raw);
#pragma unroll
                for (int k = 0; k < V; ++k) {
                    const A x = widen<Tin>(el[k]);
                    if (first)
                        acc[k] = x;
                    else if (a.op == MegRay::MEGRAY_SUM)
                        acc[k] = combine<MegRay::MEGRAY_SUM, A>(acc[k], x);
                    else if (a.op == MegRay::MEGRAY_MAX)
                        acc[k] = combine<MegRay::MEGRAY_MAX, A>(acc[k], x);
                    else
                        acc[k] = combine<MegRay::MEGRAY_MIN, A>(acc[k], x);
                }
                first = false;
            }
            if (!ok || first)
                break;
            Tout o[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                if (do_scale)
                    acc[k] = static_cast<A>(acc[k] * static_cast<A>(a.scale));
                o[k] = narrow<Tout, A>(acc[k]);
            }
            const uint32_t nel = valid / sizeof(Tin);
            Tout* dst = reinterpret_cast<Tout*>(out) + u * V;
            constexpr int OB = V * sizeof(Tout);
            if (nel == V && (reinterpret_cast<uintptr_t>(dst) & (OB >= 16 ? 15 : 7)) == 0) {
                if (OB >= 16) {
#pragma unroll
                    for (int w = 0; w < OB / 16; ++w)
                        reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(o)[w];
                } else {
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
                }
            } else {
                for (uint32_t k = 0; k < nel; ++k)
                    dst[k] = o[k];
            }
        }
    }
    stamp(c, 2);
    // rooted operations: every peer has started this call, so it has finished the previous one on
    // these slots' other parity, which the next call will overwrite
    if (a.tokens && blockIdx.x == 0 && threadIdx.x < static_cast<unsigned>(n) && static_cast<int>(threadIdx.x) != rank) {
        const uint32_t* tok = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + a.token_off) + threadIdx.x * 2;
        uint32_t spins = 0;
        uint64_t t0 = 0;
        for (;;) {
            uint32_t v;
            asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(tok) : "memory");
            if (v == a.seq)
                break;
            if ((++spins & 255) == 0) {
                const uint64_t now = globaltimer_ns();
                if (t0 == 0)
                    t0 = now;
                else if (now - t0 > c.timeout_ns) {
                    FAIL_WITH(c, kStatusTimeout, 0);
                    break;
                }
            }
        }
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

// The buffers of one call as every rank addresses them here, and what the kernel found out
// about them (shared memory, filled once per CTA after the first barrier).
struct CallBufs {
    const char* in[kMaxRanks];
    char* out[kMaxRanks];
    uint64_t in_off, out_off;  // heap offsets when in_sym / out_sym
    int in_sym, out_sym;       // every rank's buffer lies in its heap at one and the same offset
    int in_vec, out_vec;       // every rank's buffer is 16-byte aligned
};

// Ranks in separate processes name a buffer as (entry of the allocation in the owner's export
// log, offset).  The helper thread of this rank maps every entry that appears in a peer's log
// and stores the address in the import table; an entry that is not there yet is waited for.
__device__ __forceinline__ bool imported_address(const DirectArgs& a, int q, uint64_t word, char** out) {
    const CommonArgs& c = a.c;
    const uint32_t entry = static_cast<uint32_t>(word >> 48);
    const uint64_t off = word & ((1ull << 48) - 1);
    *out = nullptr;
    if (entry == kWordEntryNull)
        return true;
    if (entry == kWordEntryHeap) {
        *out = c.peers.heap[q] + off;
        return true;
    }
    if (entry >= kImportEntries || a.import_table == nullptr) {
        FAIL_WITH(c, static_cast<int>(MegRay::MEGRAY_INVALID_ARGUMENT), (static_cast<uint64_t>(q) << 32) | entry);
        return false;
    }
    const uint64_t* slot = a.import_table + static_cast<uint64_t>(q) * kImportEntries + entry;
    uint32_t spins = 0;
    uint64_t t0 = 0;
    for (;;) {
        uint64_t base;
        asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(base) : "l"(slot) : "memory");
        if (base > 1) {
            *out = reinterpret_cast<char*>(base) + off;
            return true;
        }
        if (base == 1) {  // the owner's memory could not be mapped into this process
            FAIL_WITH(c, static_cast<int>(MegRay::MEGRAY_CUDA_ERR), (static_cast<uint64_t>(q) << 32) | entry);
            return false;
        }
        if ((++spins & 63) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > c.timeout_ns) {
                FAIL_WITH(c, kStatusTimeout, (4ull << 32) | (static_cast<uint64_t>(q) << 16) | entry);  // 4: import table
                return false;
            }
        }
        __nanosleep(200);
    }
}

// The first barrier of a single-pass kernel: every rank has started this call, so whatever ran
// before it on that rank's stream is complete.  With `exchange` it is the buffer addresses
// themselves that say so: thread q stores this rank's pair into slot [parity][rank] of rank q's
// pad as four flagged words (32 payload bits + the epoch, each word written atomically), and
// polls slot [parity][q] of its own pad until all four carry this call's epoch.  No fence and no
// separate flag: nothing written by this kernel has to be visible yet.  (Every CTA stores the
// same words.  A slot was last used two calls ago, and the end barrier of the call in between
// keeps any rank from running that far ahead.)
__device__ __forceinline__ bool first_barrier(const DirectArgs& a, uint32_t target, CallBufs* cb) {
    const CommonArgs& c = a.c;
    const int n = c.nranks;
    __syncthreads();
    int ok = 1;
    if (threadIdx.x < static_cast<unsigned>(n)) {
        const int q = threadIdx.x;
        if (a.exchange) {
            char* theirs = c.peers.heap[q] + kExchangeOff + (a.parity * kMaxRanks + c.rank) * 32;
            const uint64_t pi = a.in_word, po = a.out_word;
            st_ll_v4(theirs, static_cast<uint32_t>(pi), static_cast<uint32_t>(pi >> 32), target);
            st_ll_v4(theirs + 16, static_cast<uint32_t>(po), static_cast<uint32_t>(po >> 32), target);
            const char* got = c.peers.heap[c.rank] + kExchangeOff + (a.parity * kMaxRanks + q) * 32;
            uint32_t spins = 0;
            uint64_t t0 = 0;
            cb->in[q] = nullptr;
            cb->out[q] = nullptr;
            for (;;) {
                const uint4 x = ld_ll_v4(got), y = ld_ll_v4(got + 16);
                if (x.y == target && x.w == target && y.y == target && y.w == target) {
                    const uint64_t wi = static_cast<uint64_t>(x.x) | (static_cast<uint64_t>(x.z) << 32);
                    const uint64_t wo = static_cast<uint64_t>(y.x) | (static_cast<uint64_t>(y.z) << 32);
                    if (q == c.rank) {
                        cb->in[q] = static_cast<const char*>(a.in_local);
                        cb->out[q] = static_cast<char*>(a.out_local);
                    } else if (a.exchange == 2) {
                        char* pin = nullptr;
                        char* pout = nullptr;
                        if (!imported_address(a, q, wi, &pin) || !imported_address(a, q, wo, &pout))
                            ok = 0;
                        cb->in[q] = pin;
                        cb->out[q] = pout;
                    } else {
                        cb->in[q] = reinterpret_cast<const char*>(wi);
                        cb->out[q] = reinterpret_cast<char*>(wo);
                    }
                    break;
                }
                if ((++spins & 63) == 0) {
                    const uint64_t now = globaltimer_ns();
                    if (t0 == 0)
                        t0 = now;
                    else if (now - t0 > c.timeout_ns) {
                        ok = 0;
                        FAIL_WITH(c, kStatusTimeout, (5ull << 32) | static_cast<uint64_t>(q));  // 5: a peer's buffer words
                        break;
                    }
                }
                poll_backoff(c, spins);
            }
        } else {
            uint32_t* at_peer = reinterpret_cast<uint32_t*>(c.peers.heap[q] + c.flag_off) + blockIdx.x * kMaxRanks + c.rank;
            st_release_sys(at_peer, target);
            const uint32_t* mine = reinterpret_cast<const uint32_t*>(c.peers.heap[c.rank] + c.flag_off) +
                                   blockIdx.x * kMaxRanks + q;
            ok = wait_flag_reached(c, mine, target) ? 1 : 0;
            cb->in[q] = a.in_base[q];
            cb->out[q] = a.out_base[q];
            if (q == c.rank) {  // buffers that only this rank touches need not be peer-addressable
                if (a.in_local != nullptr)
                    cb->in[q] = static_cast<const char*>(a.in_local);
                if (a.out_local != nullptr)
                    cb->out[q] = static_cast<char*>(a.out_local);
            }
        }
    }
    if (__syncthreads_and(ok) == 0)
        return false;
    if (threadIdx.x == 0) {
        uint64_t in_or = 0, out_or = 0;
        int in_sym = 1, out_sym = 1;
        const uint64_t in_off0 = static_cast<uint64_t>(cb->in[0] - c.peers.heap[0]);
        const uint64_t out_off0 = static_cast<uint64_t>(cb->out[0] - c.peers.heap[0]);
        for (int q = 0; q < n; ++q) {
            in_or |= reinterpret_cast<uint64_t>(cb->in[q]);
            out_or |= reinterpret_cast<uint64_t>(cb->out[q]);
            if (static_cast<uint64_t>(cb->in[q] - c.peers.heap[q]) != in_off0)
                in_sym = 0;
            if (static_cast<uint64_t>(cb->out[q] - c.peers.heap[q]) != out_off0)
                out_sym = 0;
        }
        cb->in_off = in_off0;
        cb->out_off = out_off0;
        cb->in_sym = in_sym && in_off0 < a.heap_bytes;
        cb->out_sym = out_sym && out_off0 < a.heap_bytes;
        cb->in_vec = (in_or & 15) == 0;
        cb->out_vec = (out_or & 15) == 0;
    }
    __syncthreads();
    return true;
}

// Reduce `nelem` elements: element i of the range is element i of in[q] + in_byte0 for every rank
// q; they are combined in rank order, scaled and cast.  The result goes to `single` + i (one
// destination) or, when `single` is null, to out[q] + out_byte0 + i of every rank.  `vec`: every
// address involved is 16-byte aligned, so the 16-byte path applies; otherwise element by element.
template <typename Tin, typename Tout, int OP, bool NVLS>
__device__ __forceinline__ void direct_reduce_range(const Guard& g, const DirectArgs& a, const CallBufs& cb,
                                                    uint64_t in_byte0, uint64_t out_byte0, uint64_t nelem,
                                                    char* single, bool vec, bool mc_in, bool mc_out) {
    using A = typename Acc<Tin>::type;
#ifdef MEGRAY_DEBUG_BOUNDS
    if (nelem == 0)
        return;
    for (int q = 0; q < a.c.nranks; ++q) {
        if (!GUARD_OK(g, cb.in[q] + in_byte0, nelem * sizeof(Tin)))
            return;
        if (single == nullptr && !GUARD_OK(g, cb.out[q] + out_byte0, nelem * sizeof(Tout)))
            return;
    }
    if (single != nullptr && !GUARD_OK(g, single, nelem * sizeof(Tout)))
        return;
#endif
    constexpr int V = 16 / sizeof(Tin);
    constexpr int OB = V * sizeof(Tout);
    const int n = a.c.nranks;
    const bool do_scale = IsFloatAcc<A>::value && OP == MegRay::MEGRAY_SUM && a.scale != 1.0f;
    const uint64_t nvec = vec ? nelem / V : 0;
    // U independent vectors per thread and iteration: all their loads are issued before the
    // first use, which is what keeps enough bytes in flight to fill the links
    constexpr int U = NVLS ? 4 : 2;
    for (uint64_t i0 = threadIdx.x; i0 < nvec; i0 += static_cast<uint64_t>(U) * blockDim.x) {
        A acc[U][V];
        if (NVLS && mc_in) {
            uint4 raw[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
                if (i < nvec)
                    raw[u] = mc_ld_reduce<Tin, OP>(a.mc_base + cb.in_off + in_byte0 + i * 16);
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
                        raw[u][q] = ld_cg_v4(cb.in[q] + in_byte0 + i * 16);
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
            if (single != nullptr) {
                char* dst = single + i * OB;
                if (OB >= 16) {
#pragma unroll
                    for (int w = 0; w < OB / 16; ++w)
                        reinterpret_cast<uint4*>(dst)[w] = reinterpret_cast<const uint4*>(o)[w];
                } else {
                    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(o);
                }
            } else if (NVLS && mc_out) {
                char* dst = a.mc_base + cb.out_off + out_byte0 + i * OB;
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
                        char* dst = cb.out[(a.c.rank + q) % n] + out_byte0 + i * OB;
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
    // what the 16-byte path left (fewer than V elements, or everything when something is
    // unaligned): plain element accesses
    for (uint64_t i = nvec * V + threadIdx.x; i < nelem; i += blockDim.x) {
        A acc = widen<Tin>(__ldcg(reinterpret_cast<const Tin*>(cb.in[0] + in_byte0) + i));
        for (int q = 1; q < n; ++q)
            acc = combine<OP, A>(acc, widen<Tin>(__ldcg(reinterpret_cast<const Tin*>(cb.in[q] + in_byte0) + i)));
        if (do_scale)
            acc = static_cast<A>(acc * static_cast<A>(a.scale));
        const Tout o = narrow<Tout, A>(acc);
        if (single != nullptr) {
            reinterpret_cast<Tout*>(single)[i] = o;
        } else {
            for (int q = 0; q < n; ++q)
                reinterpret_cast<Tout*>(cb.out[q] + out_byte0)[i] = o;
        }
    }
}

// Copy [0, nbytes) of `src` to the same range of up to n destinations, reading the source once:
// every 16-byte vector goes to all destinations before the next one is touched, so all links
// carry traffic at every moment (dst[j] == nullptr is skipped).
__device__ __forceinline__ void cta_fanout(const Guard& g, char* const* dst, int ndst, const char* src,
                                           uint64_t nbytes, bool vec) {
    if (nbytes == 0)
        return;
#ifdef MEGRAY_DEBUG_BOUNDS
    if (!GUARD_OK(g, src, nbytes))
        return;
    for (int j = 0; j < ndst; ++j)
        if (dst[j] != nullptr && !GUARD_OK(g, dst[j], nbytes))
            return;
#endif
    if (!vec || (nbytes & 15)) {
        for (int j = 0; j < ndst; ++j)
            if (dst[j] != nullptr)
                cta_copy(g, dst[j], src, nbytes);
        return;
    }
    const uint64_t nv = nbytes / 16;
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    constexpr int U = 4;
    for (uint64_t i0 = threadIdx.x; i0 < nv; i0 += static_cast<uint64_t>(U) * blockDim.x) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
            if (i < nv)
                v[u] = __ldcg(s4 + i);
        }
#pragma unroll
        for (int j = 0; j < kMaxRanks; ++j) {
            if (j < ndst && dst[j] != nullptr) {
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
                    if (i < nv)
                        reinterpret_cast<uint4*>(dst[j])[i] = v[u];
                }
            }
        }
    }
}

// Copy [0, nbytes) of src[j] to dst[j] for up to n pairs, one vector of every pair in flight at
// a time (all_to_all, scatter: a different source chunk for every destination).
__device__ __forceinline__ void cta_pairs(const Guard& g, char* const* dst, const char* const* src, int npairs,
                                          uint64_t nbytes, bool vec) {
    if (nbytes == 0)
        return;
#ifdef MEGRAY_DEBUG_BOUNDS
    for (int j = 0; j < npairs; ++j)
        if (dst[j] != nullptr && (!GUARD_OK(g, dst[j], nbytes) || !GUARD_OK(g, src[j], nbytes)))
            return;
#endif
    if (!vec || (nbytes & 15)) {
        for (int j = 0; j < npairs; ++j)
            if (dst[j] != nullptr)
                cta_copy(g, dst[j], src[j], nbytes);
        return;
    }
    const uint64_t nv = nbytes / 16;
    constexpr int U = 2;
    for (uint64_t i0 = threadIdx.x; i0 < nv; i0 += static_cast<uint64_t>(U) * blockDim.x) {
        uint4 v[U][kMaxRanks];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j)
                if (j < npairs && dst[j] != nullptr && i < nv)
                    v[u][j] = __ldcg(reinterpret_cast<const uint4*>(src[j]) + i);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + static_cast<uint64_t>(u) * blockDim.x;
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j)
                if (j < npairs && dst[j] != nullptr && i < nv)
                    reinterpret_cast<uint4*>(dst[j])[i] = v[u][j];
        }
    }
}

template <typename Tin, typename Tout, bool NVLS>
__global__ void __launch_bounds__(512) direct_family_kernel(const DirectArgs a) {
    __shared__ CallBufs cb;
    __shared__ int s_ok;
    __shared__ uint32_t s_round[16];  // a root's storing warps: rounds issued (see warp_round_done)
    const CommonArgs& c = a.c;
    const int n = c.nranks, rank = c.rank;
    constexpr uint64_t V = 16 / sizeof(Tin);
    if (threadIdx.x < 16)
        s_round[threadIdx.x] = 0;
    if (threadIdx.x == 0)
        s_ok = 1;
    uint32_t epoch = c.epoch;
    stamp(c, 0);
    // inputs are final / outputs may be overwritten on every rank
    if (!first_barrier(a, ++epoch, &cb))
        return;
    stamp(c, 1);
    Guard g = make_guard(c);
#ifdef MEGRAY_DEBUG_BOUNDS
    for (int q = 0; q < n; ++q) {
        g.peer_in[q] = cb.in[q];
        g.peer_out[q] = cb.out[q];
    }
#endif
    const char* const my_in = cb.in[rank];
    char* const my_out = cb.out[rank];
    if (a.kind == DIRECT_ALL_GATHER || a.kind == DIRECT_GATHER) {
        // this rank's block into slot `rank` of every output (all_gather) or of the root's (gather)
        const uint64_t bytes = a.len * sizeof(Tin);
        const uint64_t per_cta = round_up_u64((bytes + gridDim.x - 1) / gridDim.x, 16);
        const uint64_t b = min(bytes, per_cta * blockIdx.x), e = min(bytes, b + per_cta);
        const bool vec = cb.out_vec && ((reinterpret_cast<uint64_t>(my_in) | bytes) & 15) == 0;
        if (a.kind == DIRECT_GATHER) {
            cta_copy(g, cb.out[a.root] + rank * bytes + b, my_in + b, e - b);
        } else if (NVLS && cb.out_sym && vec && GUARD_OK(g, my_out + rank * bytes + b, e - b) &&
                   GUARD_OK(g, my_in + b, e - b)) {
            char* dst = a.mc_base + cb.out_off + rank * bytes;
            const uint64_t nv = (e - b) / 16;
            for (uint64_t i = threadIdx.x; i < nv; i += blockDim.x)
                mc_st_v4(dst + b + i * 16, ld_cg_v4(my_in + b + i * 16));
        } else {
            char* dst[kMaxRanks];
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j)
                dst[j] = j < n ? cb.out[(rank + 1 + j) % n] + rank * bytes + b : nullptr;
            cta_fanout(g, dst, n, my_in + b, e - b, vec);
        }
    } else if (a.kind == DIRECT_ALL_TO_ALL || a.kind == DIRECT_SCATTER) {
        // chunk q of the input into slot `rank` of rank q's output (all_to_all) or into rank q's
        // output (scatter, root only), starting with rank + 1
        const uint64_t bytes = a.len * sizeof(Tin);
        const uint64_t per_cta = round_up_u64((bytes + gridDim.x - 1) / gridDim.x, 16);
        const uint64_t b = min(bytes, per_cta * blockIdx.x), e = min(bytes, b + per_cta);
        if (a.kind == DIRECT_ALL_TO_ALL || rank == a.root) {
            const uint64_t slot = a.kind == DIRECT_ALL_TO_ALL ? rank * bytes : 0;
            const bool vec = cb.out_vec && ((reinterpret_cast<uint64_t>(my_in) | bytes) & 15) == 0;
            char* dst[kMaxRanks];
            const char* src[kMaxRanks];
#pragma unroll
            for (int j = 0; j < kMaxRanks; ++j) {
                const int q = (rank + 1 + j) % n;
                dst[j] = j < n ? cb.out[q] + slot + b : nullptr;
                src[j] = j < n ? my_in + q * bytes + b : nullptr;
            }
            cta_pairs(g, dst, src, n, e - b, vec);
        }
    } else if (a.kind == DIRECT_BROADCAST) {
        const uint64_t S = a.len * sizeof(Tin);
        const int root = a.root;
        if (a.bcast_pull && n >= 2) {
            // Broadcast by loads alone.  The message is cut into n - 1 slices, one per non-root rank.
            // Chunk by chunk, a rank loads its own slice from the root's input into its output,
            // raises the chunk counter that every other non-root rank keeps for (CTA, this rank),
            // and then loads the same chunk of the other slices from their owners' outputs as
            // their counters arrive.  Nobody stores to a peer but counters; the root only serves
            // loads (and copies its input to its own output).
            const BcastPlan pl = bcast_plan(S, n, gridDim.x, a.chunk_bytes);
            const uint64_t sb = pl.per_cta * blockIdx.x;  // this CTA's share of every slice
            auto chunk_range = [&](int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
                const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
                const uint64_t L = s0 >= S ? 0 : min(pl.slice, S - s0);
                *lo = min(L, sb + static_cast<uint64_t>(k) * a.chunk_bytes);
                *hi = min(L, min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * a.chunk_bytes));
            };
            if (rank == root) {
                if (my_out != my_in) {
                    for (int v = 0; v < n - 1; ++v) {
                        const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
                        const uint64_t L = s0 >= S ? 0 : min(pl.slice, S - s0);
                        const uint64_t lo = min(L, sb), hi = min(L, sb + pl.per_cta);
                        if (hi > lo)
                            cta_copy(g, my_out + s0 + lo, my_in + s0 + lo, hi - lo);
                    }
                }
            } else {
                const int v = (rank - root - 1 + n) % n;  // this rank's slice
                const char* root_in = cb.in[root];
                for (uint32_t k = 0; k < pl.chunks; ++k) {
                    uint64_t lo, hi;
                    chunk_range(v, k, &lo, &hi);
                    if (hi > lo)
                        cta_copy(g, my_out + v * pl.slice + lo, root_in + v * pl.slice + lo, hi - lo);
                    __syncthreads();  // the chunk is stored (locally)
                    if (threadIdx.x < static_cast<unsigned>(n - 1)) {
                        const int u = static_cast<int>(threadIdx.x);  // another slice, and its owner
                        const int m = (root + 1 + u) % n;
                        if (u != v) {
                            if (hi > lo)
                                st_release_sys(reinterpret_cast<uint32_t*>(c.peers.heap[m] + kCreditOff) +
                                                       blockIdx.x * kMaxRanks + rank,
                                               a.chunk_base + k + 1);
                            uint64_t lo2, hi2;
                            chunk_range(u, k, &lo2, &hi2);
                            const uint32_t* ready = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kCreditOff) +
                                                    blockIdx.x * kMaxRanks + m;
                            if (hi2 > lo2 && !wait_flag_reached(c, ready, a.chunk_base + k + 1, 2))
                                s_ok = 0;
                        }
                    }
                    __syncthreads();
                    if (!s_ok)
                        return;
                    for (int uu = 0; uu < n - 1; ++uu) {
                        const int u = (uu + static_cast<int>(k) + static_cast<int>(blockIdx.x)) % (n - 1);
                        if (u == v)
                            continue;
                        const int m = (root + 1 + u) % n;
                        uint64_t lo2, hi2;
                        chunk_range(u, k, &lo2, &hi2);
                        if (hi2 > lo2)
                            cta_copy(g, my_out + u * pl.slice + lo2, cb.out[m] + u * pl.slice + lo2, hi2 - lo2);
                    }
                }
            }
        } else if (n <= 2) {
            // nobody to forward to: the root stores its share to the other rank (and to itself)
            const uint64_t per_cta = round_up_u64((S + gridDim.x - 1) / gridDim.x, 16);
            const uint64_t b = min(S, per_cta * blockIdx.x), e = min(S, b + per_cta);
            if (rank == root) {
                // every vector is loaded once and stored to the other rank and to the root's own output
                char* dst[kMaxRanks];
#pragma unroll
                for (int j = 0; j < kMaxRanks; ++j)
                    dst[j] = nullptr;
                dst[0] = n == 2 ? cb.out[1 - rank] + b : nullptr;
                dst[1] = my_out != my_in ? my_out + b : nullptr;
                const bool vec = ((reinterpret_cast<uint64_t>(my_in + b) | reinterpret_cast<uint64_t>(dst[0]) |
                                   reinterpret_cast<uint64_t>(dst[1])) & 15) == 0;
                cta_fanout(g, dst, 2, my_in + b, e - b, vec);
            }
        } else {
            const BcastPlan pl = bcast_plan(S, n, gridDim.x, a.chunk_bytes);
            const uint64_t sb = pl.per_cta * blockIdx.x;  // this CTA's share of every slice
            // bytes [lo, hi) of slice v that chunk k of this CTA covers (relative to the slice)
            auto chunk_range = [&](int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
                const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
                const uint64_t L = s0 >= S ? 0 : min(pl.slice, S - s0);
                *lo = min(L, sb + static_cast<uint64_t>(k) * a.chunk_bytes);
                *hi = min(L, min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * a.chunk_bytes));
            };
            if (rank == root) {
                // The last warp only announces; the other warps store round after round (chunk k of
                // every slice, and the same bytes into the root's own output) without ever waiting
                // for a store to be acknowledged or for the announcing warp.  Each storing warp
                // counts the rounds it has issued in shared memory; the announcing warp takes the
                // minimum and, whenever that has grown, publishes it to all forwarders with one
                // warp-wide releasing store (lane v to the forwarder of slice v).  The release waits
                // for the stores issued so far, which under load takes as long as several rounds:
                // the next announcement then simply covers all of them.
                const unsigned ncopy = blockDim.x - 32;
                const bool announcer = threadIdx.x >= ncopy;
                if (!announcer) {
                    for (uint32_t k = 0; k < pl.chunks; ++k) {
                        // slice by slice, starting with a different one in every round and in every
                        // CTA: at any moment the CTAs store to all destinations alike (all of them
                        // storing to one destination at a time would be limited by that GPU's link)
                        for (int vv = 0; vv < n - 1; ++vv) {
                            const int v = (vv + static_cast<int>(k) + static_cast<int>(blockIdx.x)) % (n - 1);
                            const int j = (root + 1 + v) % n;
                            uint64_t lo, hi;
                            chunk_range(v, k, &lo, &hi);
                            if (hi > lo) {
                                cta_copy_part(g, cb.out[j] + v * pl.slice + lo, my_in + v * pl.slice + lo, hi - lo,
                                              threadIdx.x, ncopy);
                                if (my_out != my_in)
                                    cta_copy_part(g, my_out + v * pl.slice + lo, my_in + v * pl.slice + lo, hi - lo,
                                                  threadIdx.x, ncopy);
                            }
                        }
                        warp_round_done(s_round, k + 1);
                    }
                } else {
                    uint32_t published = 0;
                    while (published < pl.chunks) {
                        const uint32_t m = rounds_done_by_all(s_round, ncopy / 32);
                        if (m > published) {
                            const int v = static_cast<int>(threadIdx.x - ncopy);
                            if (v < n - 1) {
                                const int j = (root + 1 + v) % n;
                                st_release_sys(reinterpret_cast<uint32_t*>(c.peers.heap[j] + kChunkFlagOff) + blockIdx.x,
                                               a.chunk_base + m);
                            }
                            published = m;
                        } else {
                            __nanosleep(100);
                        }
                    }
                }
            } else {
                const int v = (rank - root - 1 + n) % n;  // the slice this rank forwards
                const uint32_t* my_flag =
                        reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kChunkFlagOff) + blockIdx.x;
                for (uint32_t k = 0; k < pl.chunks; ++k) {
                    uint64_t lo, hi;
                    chunk_range(v, k, &lo, &hi);
                    if (hi <= lo)
                        continue;  // (uniform over the CTA) nothing to wait for, nothing to forward
                    if (threadIdx.x == 0)
                        s_ok = wait_flag_reached(c, my_flag, a.chunk_base + k + 1, 2) ? 1 : 0;
                    __syncthreads();
                    if (!s_ok)
                        return;
                    if (n > 2) {
                        char* dst[kMaxRanks];
                        const char* src = my_out + v * pl.slice + lo;
                        bool vec = (reinterpret_cast<uint64_t>(src) & 15) == 0;
#pragma unroll
                        for (int j = 0; j < kMaxRanks; ++j) {
                            const int m = (rank + 1 + j) % n;
                            dst[j] = (j < n - 1 && m != root) ? cb.out[m] + v * pl.slice + lo : nullptr;
                            if (dst[j] != nullptr && (reinterpret_cast<uint64_t>(dst[j]) & 15))
                                vec = false;
                        }
                        cta_fanout(g, dst, n - 1, src, hi - lo, vec);
                    }
                    __syncthreads();  // s_ok is rewritten in the next round
                }
            }
        }
    } else if (a.kind == DIRECT_REDUCE && a.stage_slots > 0 && n > 2 && a.reduce_mode == 3) {
        // Reduce in steps, loads only, with nothing but the per-CTA barrier between the steps.  One
        // slice per non-root rank; a CTA's share of a slice is cut into stage_slots pieces.  In
        // step t every reducer loads piece t of its slice from every rank and stores the reduced
        // piece into one of two slots in its own heap, while the root loads piece t - 1 of every
        // slice from the reducers' other slot into its output; a barrier ends the step.  The
        // reducers' work of one step and the root's work on the step before run side by side, so
        // the whole takes (pieces + 1) / pieces of the time of the loads alone.
        const int root = a.root;
        const uint32_t pieces = a.stage_slots;
        const uint64_t se = round_up_u64((a.len + n - 2) / (n - 1), V);
        const uint64_t per_cta = round_up_u64((se + gridDim.x - 1) / gridDim.x, V);
        const uint64_t piece_el = a.chunk_bytes / sizeof(Tin);
        const uint64_t sb = per_cta * blockIdx.x;
        auto piece_range = [&](int v, uint32_t t, uint64_t* lo, uint64_t* hi) {
            const uint64_t s0 = static_cast<uint64_t>(v) * se;
            const uint64_t L = s0 >= a.len ? 0 : min(se, a.len - s0);
            *lo = min(L, sb + static_cast<uint64_t>(t) * piece_el);
            *hi = min(L, min(sb + per_cta, sb + static_cast<uint64_t>(t + 1) * piece_el));
        };
        auto slot_off = [&](uint32_t t) {
            return a.stage_off + (static_cast<uint64_t>(blockIdx.x) * 2 + (t & 1)) * a.chunk_bytes;
        };
        for (uint32_t t = 0; t <= pieces; ++t) {
            if (rank != root && t < pieces) {
                const int v = (rank - root - 1 + n) % n;
                uint64_t lo, hi;
                piece_range(v, t, &lo, &hi);
                if (hi > lo) {
                    const uint64_t in_byte0 = (v * se + lo) * sizeof(Tin);
                    char* single = c.peers.heap[rank] + slot_off(t);
                    const bool vec = cb.in_vec && (in_byte0 & 15) == 0;
                    switch (a.op) {
                        case MegRay::MEGRAY_SUM:
                            direct_reduce_range<Tin, Tout, MegRay::MEGRAY_SUM, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec,
                                                                                      false, false);
                            break;
                        case MegRay::MEGRAY_MAX:
                            direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MAX, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec,
                                                                                      false, false);
                            break;
                        default:
                            direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MIN, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec,
                                                                                      false, false);
                    }
                }
            }
            if (rank == root && t >= 1) {
                for (int vv = 0; vv < n - 1; ++vv) {
                    const int v = (vv + static_cast<int>(blockIdx.x)) % (n - 1);
                    const int j = (root + 1 + v) % n;
                    uint64_t lo, hi;
                    piece_range(v, t - 1, &lo, &hi);
                    if (hi > lo)
                        cta_copy(g, my_out + (v * se + lo) * sizeof(Tout), c.peers.heap[j] + slot_off(t - 1),
                                 (hi - lo) * sizeof(Tout));
                }
            }
            // the reduced pieces of this step are stored / the slots read in this step are free again
            if (t < pieces && !cta_barrier(c, ++epoch))
                return;
        }
    } else if (a.kind == DIRECT_REDUCE && a.stage_slots > 0 && n > 1 && a.reduce_mode == 2) {
        // Reduce by loads alone (the fastest way to move bytes that was measured here: a kernel
        // that only loads from its peers sustains more than one that loads and stores to them).
        // One slice per non-root rank.  The reducer of a slice loads it from every rank and stores
        // the reduced chunk into a slot in its own heap, then raises the chunk counter the root
        // keeps for (CTA, reducer); the root waits for the counters, loads the chunks into its
        // output and raises the consumed-chunk counter in the reducer's pad, which frees the slot.
        // Every link carries one message's worth each way, and nobody stores to a peer but flags.
        const int root = a.root;
        const ReducePlan pl = reduce_plan(a.len, n, gridDim.x, a.chunk_bytes, sizeof(Tin));
        const uint64_t sb = pl.per_cta * blockIdx.x;
        auto chunk_range = [&](int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
            const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
            const uint64_t L = s0 >= a.len ? 0 : min(pl.slice, a.len - s0);
            *lo = min(L, sb + static_cast<uint64_t>(k) * pl.chunk_el);
            *hi = min(L, min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * pl.chunk_el));
        };
        auto slot_off = [&](uint32_t k) {
            return a.stage_off + (static_cast<uint64_t>(blockIdx.x) * a.stage_slots + k % a.stage_slots) * a.chunk_bytes;
        };
        if (rank == root) {
            for (uint32_t k = 0; k < pl.chunks; ++k) {
                // chunk k of every slice is ready?
                if (threadIdx.x < static_cast<unsigned>(n - 1)) {
                    const int v = static_cast<int>(threadIdx.x);
                    const int j = (root + 1 + v) % n;
                    uint64_t lo, hi;
                    chunk_range(v, k, &lo, &hi);
                    const uint32_t* ready = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kCreditOff) +
                                            blockIdx.x * kMaxRanks + j;
                    if (hi > lo && !wait_flag_reached(c, ready, a.chunk_base + k + 1, 2))
                        s_ok = 0;
                }
                __syncthreads();
                if (!s_ok)
                    return;
                for (int vv = 0; vv < n - 1; ++vv) {
                    const int v = (vv + static_cast<int>(k) + static_cast<int>(blockIdx.x)) % (n - 1);
                    const int j = (root + 1 + v) % n;
                    uint64_t lo, hi;
                    chunk_range(v, k, &lo, &hi);
                    if (hi > lo)
                        cta_copy(g, my_out + (v * pl.slice + lo) * sizeof(Tout), c.peers.heap[j] + slot_off(k),
                                 (hi - lo) * sizeof(Tout));
                }
                __syncthreads();  // every thread has loaded its part of the slots
                if (threadIdx.x < static_cast<unsigned>(n - 1)) {
                    const int v = static_cast<int>(threadIdx.x);
                    const int j = (root + 1 + v) % n;
                    uint64_t lo, hi;
                    chunk_range(v, k, &lo, &hi);
                    if (hi > lo) {
                        uint32_t* consumed = reinterpret_cast<uint32_t*>(c.peers.heap[j] + kChunkFlagOff) + blockIdx.x;
                        asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(consumed), "r"(a.chunk_base + k + 1) : "memory");
                    }
                }
            }
        } else {
            const int v = (rank - root - 1 + n) % n;  // the slice this rank reduces
            const uint32_t* consumed = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kChunkFlagOff) + blockIdx.x;
            uint32_t* ready = reinterpret_cast<uint32_t*>(c.peers.heap[root] + kCreditOff) + blockIdx.x * kMaxRanks + rank;
            for (uint32_t k = 0; k < pl.chunks; ++k) {
                uint64_t lo, hi;
                chunk_range(v, k, &lo, &hi);
                if (hi <= lo)
                    continue;  // (uniform over the CTA)
                if (k >= a.stage_slots) {
                    // the slot still holds chunk k - stage_slots until the root has loaded it
                    if (threadIdx.x == 0)
                        s_ok = wait_flag_reached(c, consumed, a.chunk_base + (k - a.stage_slots) + 1, 3) ? 1 : 0;
                    __syncthreads();
                    if (!s_ok)
                        return;
                }
                const uint64_t in_byte0 = (v * pl.slice + lo) * sizeof(Tin);
                char* single = c.peers.heap[rank] + slot_off(k);
                const bool vec = cb.in_vec && (in_byte0 & 15) == 0;
                switch (a.op) {
                    case MegRay::MEGRAY_SUM:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_SUM, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec, false,
                                                                                  false);
                        break;
                    case MegRay::MEGRAY_MAX:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MAX, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec, false,
                                                                                  false);
                        break;
                    default:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MIN, false>(g, a, cb, in_byte0, 0, hi - lo, single, vec, false,
                                                                                  false);
                }
                __syncthreads();  // the whole chunk is stored (locally)
                if (threadIdx.x == 0)
                    st_release_sys(ready, a.chunk_base + k + 1);
            }
        }
    } else if (a.kind == DIRECT_REDUCE && a.stage_slots > 0 && n > 1) {
        // Reduce with the root's input pushed.  One slice per non-root rank, as below, but the
        // reducer of a slice does not load the root's part over NVLink: the root stores it, chunk
        // by chunk, into staging slots in the reducer's heap (the root has nothing else to do).
        // Every GPU then issues about one message's worth of transfers (the root its input, a
        // reducer the other non-root inputs of its slice plus its result) instead of the reducers
        // issuing all of them.  CTA b of the root feeds CTA b of every reducer; a slot is written
        // again only after its reader has reported the chunk that was in it as consumed.
        const int root = a.root;
        const ReducePlan pl = reduce_plan(a.len, n, gridDim.x, a.chunk_bytes, sizeof(Tin));
        const uint64_t sb = pl.per_cta * blockIdx.x;  // this CTA's share of every slice (elements)
        // elements [lo, hi) of slice v that chunk k of this CTA covers (relative to the slice)
        auto chunk_range = [&](int v, uint32_t k, uint64_t* lo, uint64_t* hi) {
            const uint64_t s0 = static_cast<uint64_t>(v) * pl.slice;
            const uint64_t L = s0 >= a.len ? 0 : min(pl.slice, a.len - s0);
            *lo = min(L, sb + static_cast<uint64_t>(k) * pl.chunk_el);
            *hi = min(L, min(sb + pl.per_cta, sb + static_cast<uint64_t>(k + 1) * pl.chunk_el));
        };
        auto slot_off = [&](uint32_t k) {
            return a.stage_off + (static_cast<uint64_t>(blockIdx.x) * a.stage_slots + k % a.stage_slots) * a.chunk_bytes;
        };
        if (rank == root) {
            // (storing warps and announcing warp as in the broadcast above)
            const unsigned ncopy = blockDim.x - 32;
            const bool announcer = threadIdx.x >= ncopy;
            if (!announcer) {
                for (uint32_t k = 0; k < pl.chunks; ++k) {
                    if (k >= a.stage_slots) {
                        // the slot still holds chunk k - stage_slots until its reducer has consumed it
                        if (threadIdx.x < static_cast<unsigned>(n - 1) && s_ok) {
                            const int j = (root + 1 + static_cast<int>(threadIdx.x)) % n;
                            const uint32_t* credit = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kCreditOff) +
                                                     blockIdx.x * kMaxRanks + j;
                            uint64_t lo, hi;
                            chunk_range(static_cast<int>(threadIdx.x), k - a.stage_slots, &lo, &hi);
                            // (a reducer reports only chunks that held something)
                            if (hi > lo && !wait_flag_reached(c, credit, a.chunk_base + (k - a.stage_slots) + 1, 3))
                                s_ok = 0;  // (status says why; the loop runs on without waiting, so the kernel ends)
                        }
                        named_bar_sync(9, ncopy);
                    }
                    for (int vv = 0; vv < n - 1; ++vv) {
                        const int v = (vv + static_cast<int>(k) + static_cast<int>(blockIdx.x)) % (n - 1);
                        const int j = (root + 1 + v) % n;
                        uint64_t lo, hi;
                        chunk_range(v, k, &lo, &hi);
                        if (hi > lo)
                            cta_copy_part(g, c.peers.heap[j] + slot_off(k), my_in + (v * pl.slice + lo) * sizeof(Tin),
                                          (hi - lo) * sizeof(Tin), threadIdx.x, ncopy);
                    }
                    warp_round_done(s_round, k + 1);
                }
            } else {
                uint32_t published = 0;
                while (published < pl.chunks) {
                    const uint32_t m = rounds_done_by_all(s_round, ncopy / 32);
                    if (m > published) {
                        const int v = static_cast<int>(threadIdx.x - ncopy);
                        if (v < n - 1) {
                            const int j = (root + 1 + v) % n;
                            st_release_sys(reinterpret_cast<uint32_t*>(c.peers.heap[j] + kChunkFlagOff) + blockIdx.x,
                                           a.chunk_base + m);
                        }
                        published = m;
                    } else {
                        __nanosleep(100);
                    }
                }
            }
        } else {
            const int v = (rank - root - 1 + n) % n;  // the slice this rank reduces
            const uint32_t* my_flag = reinterpret_cast<const uint32_t*>(c.peers.heap[rank] + kChunkFlagOff) + blockIdx.x;
            uint32_t* credit = reinterpret_cast<uint32_t*>(c.peers.heap[root] + kCreditOff) + blockIdx.x * kMaxRanks + rank;
            for (uint32_t k = 0; k < pl.chunks; ++k) {
                uint64_t lo, hi;
                chunk_range(v, k, &lo, &hi);
                if (hi <= lo)
                    continue;  // (uniform over the CTA) the root stores nothing for it either
                const uint64_t in_byte0 = (v * pl.slice + lo) * sizeof(Tin);
                const uint64_t out_byte0 = (v * pl.slice + lo) * sizeof(Tout);
                if (threadIdx.x == 0) {
                    s_ok = wait_flag_reached(c, my_flag, a.chunk_base + k + 1, 2) ? 1 : 0;
                    // the root's part of this chunk: in the slot, addressed like the other inputs
                    cb.in[root] = c.peers.heap[rank] + slot_off(k) - in_byte0;
                }
                __syncthreads();
                if (!s_ok)
                    return;
                char* single = cb.out[root] + out_byte0;
                const bool vec = cb.in_vec && (in_byte0 & 15) == 0 && (reinterpret_cast<uint64_t>(single) & 15) == 0;
                switch (a.op) {
                    case MegRay::MEGRAY_SUM:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_SUM, false>(g, a, cb, in_byte0, out_byte0, hi - lo, single,
                                                                                  vec, false, false);
                        break;
                    case MegRay::MEGRAY_MAX:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MAX, false>(g, a, cb, in_byte0, out_byte0, hi - lo, single,
                                                                                  vec, false, false);
                        break;
                    default:
                        direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MIN, false>(g, a, cb, in_byte0, out_byte0, hi - lo, single,
                                                                                  vec, false, false);
                }
                __syncthreads();  // every thread has loaded its part of the slot
                if (threadIdx.x == 0)
                    asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(credit), "r"(a.chunk_base + k + 1) : "memory");
            }
        }
    } else {
        // all_reduce: len is cut into n slices of se elements and this rank reduces slice `rank`;
        // reduce_scatter: its slice is the rank-th block of len elements; reduce: n - 1 slices, one
        // per non-root rank, so that the root's links carry only its input (out) and the result
        // (in), not a slice's operands as well
        uint64_t se, elem0, L;
        if (a.kind == DIRECT_REDUCE_SCATTER) {
            elem0 = a.len * rank;
            L = a.len;
        } else if (a.kind == DIRECT_REDUCE && n == 2) {
            // two ranks: the root loads the other rank's input and reduces into its own output
            // (loads only, like reduce_scatter; the other rank loading and storing back over the
            // same link measured a quarter slower)
            elem0 = 0;
            L = rank == a.root ? a.len : 0;
        } else if (a.kind == DIRECT_REDUCE && n > 1) {
            if (rank == a.root) {
                elem0 = 0;
                L = 0;
            } else {
                const int v = (rank - a.root - 1 + n) % n;
                se = round_up_u64((a.len + n - 2) / (n - 1), V);
                elem0 = min(a.len, se * v);
                L = min(a.len, elem0 + se) - elem0;
            }
        } else {
            se = round_up_u64((a.len + n - 1) / n, V);
            elem0 = min(a.len, se * rank);
            L = min(a.len, elem0 + se) - elem0;
        }
        const uint64_t per_cta = round_up_u64((L + gridDim.x - 1) / gridDim.x, V);
        const uint64_t b = min(L, per_cta * blockIdx.x), e = min(L, b + per_cta);
        const uint64_t in_byte0 = (elem0 + b) * sizeof(Tin);
        uint64_t out_byte0 = (elem0 + b) * sizeof(Tout);
        char* single = nullptr;
        bool vec = cb.in_vec && (in_byte0 & 15) == 0;
        if (a.kind == DIRECT_REDUCE_SCATTER) {
            single = my_out + b * sizeof(Tout);
            vec = vec && (reinterpret_cast<uint64_t>(single) & 15) == 0;
        } else if (a.kind == DIRECT_REDUCE) {
            single = cb.out[a.root] + out_byte0;
            vec = vec && (reinterpret_cast<uint64_t>(single) & 15) == 0;
        } else {
            vec = vec && cb.out_vec && (out_byte0 & 15) == 0;
        }
        const bool mc_in = NVLS && cb.in_sym && vec;
        const bool mc_out = NVLS && cb.out_sym && vec && single == nullptr;
        switch (a.op) {
            case MegRay::MEGRAY_SUM:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_SUM, NVLS>(g, a, cb, in_byte0, out_byte0, e - b, single, vec,
                                                                         mc_in, mc_out);
                break;
            case MegRay::MEGRAY_MAX:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MAX, NVLS>(g, a, cb, in_byte0, out_byte0, e - b, single, vec,
                                                                         mc_in, mc_out);
                break;
            default:
                direct_reduce_range<Tin, Tout, MegRay::MEGRAY_MIN, NVLS>(g, a, cb, in_byte0, out_byte0, e - b, single, vec,
                                                                         mc_in, mc_out);
        }
    }
    stamp(c, 2);
    // all transfers are complete before any rank uses its output or overwrites its input
    cta_barrier(c, ++epoch);
    stamp(c, 3);
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
struct LLLauncher {
    const LLArgs& a;
    int ctas, threads;
    cudaStream_t s;
    template <typename Tin, typename Tout>
    cudaError_t operator()() const {
        ll_family_kernel<Tin, Tout><<<ctas, threads, 0, s>>>(a);
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
    if (a.mc_base != nullptr &&
        (a.kind == DIRECT_ALL_REDUCE || a.kind == DIRECT_REDUCE_SCATTER || a.kind == DIRECT_REDUCE) &&
        !nvls_supports(a.in_dtype, a.out_dtype, a.op))
        return cudaErrorInvalidValue;
    if (a.kind == DIRECT_BROADCAST && (a.chunk_bytes < 16 || (a.chunk_bytes & 15)))
        return cudaErrorInvalidValue;
    return dispatch_types(a.in_dtype, a.out_dtype, DirectLauncher{a, ctas, threads, stream});
}

cudaError_t launch_ll(const LLArgs& a, int ctas, int threads, cudaStream_t stream) {
    if (ctas < 1 || ctas > kMaxCtas || threads < 32 || threads > 512 || a.c.nranks < 1 || a.c.nranks > kMaxRanks ||
        a.bytes > kLLMaxBytes || a.seq == 0)
        return cudaErrorInvalidValue;
    if (!a.reduce)  // pure data movement: the element type does not matter
        return LLLauncher{a, ctas, threads, stream}.template operator()<uint8_t, uint8_t>();
    return dispatch_types(a.in_dtype, a.out_dtype, LLLauncher{a, ctas, threads, stream});
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
