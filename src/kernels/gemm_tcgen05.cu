// Persistent warp-specialised bf16 GEMM for sm_100a on tcgen05 tensor cores.
//
//   warp 0      : TMA producer   (cp.async.bulk.tensor 2D tiles -> 128B-swizzled smem ring)
//   warp 1      : UMMA issuer    (tcgen05.mma, accumulators in TMEM)
//   warps 2..5  : epilogue       (tcgen05.ld TMEM -> registers -> fused epilogue -> swizzled
//                                 staging boxes -> TMA store; row segments for the push epilogue)
//   warps 6..9  : communication  (fused all_gather: pull the peers' shards) and, on the wide
//                                 tile, a second epilogue group
//
// Three variants of one kernel template:
//   single : one CTA per tile, tile 128 x 256 x 64, tcgen05.mma.cta_group::1 (M = 128),
//            4-stage ring of 48 KB.  Used for grouped (per-expert) row blocks.
//   pair   : a cluster of two CTAs per 256 x 256 tile, tcgen05.mma.cta_group::2 (M = 256)
//            issued by the leader CTA; each CTA stages its own 128 rows of A and its own
//            128 rows of B (so B is read from shared memory once per pair), 6-stage ring
//            of 32 KB per CTA.  Each CTA issues its own TMA loads (no multicast); their
//            byte counts complete on the leader's barrier, and the leader's commits free
//            the stage in both CTAs.
//   wide   : a CTA pair per 512 x 256 tile: two 256-row sub-tiles of A against one B tile,
//            each with its own 256-column accumulator, so every staged byte of B feeds twice
//            the math (0.75 of the pair variant's L2 -> shared-memory traffic per FLOP).
//            4-stage ring of 48 KB per CTA.
// single and pair keep two TMEM accumulators (2 x 256 columns) so the epilogue of tile i
// overlaps the main loop of tile i+1; wide uses all 512 columns for one tile and restarts
// the main loop on each sub-tile's accumulator as soon as the epilogue has drained it.
// Every wait is bounded: a wait that runs out sets the kernel's error word, all roles
// leave their loops, TMEM is freed and the kernel returns normally.
//
// The reference library (MegRay) contains no GEMM; this kernel exists for the
// fused tensor-parallel and expert-parallel entry points.
#include "gemm_tcgen05.cuh"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "launch_count.h"
#include "ptx_sm100.cuh"

namespace mgk {
namespace gemm {

using namespace mgk::ptx;

namespace {

constexpr int BM = 128;  // rows of A per CTA
constexpr int BN = 256;  // accumulator columns
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int TMEM_COLS = 512;
constexpr int NUM_THREADS = 320;   // producer, MMA, 4 epilogue warps, 4 communication warps
constexpr int COMM_THREADS = 128;
constexpr int MN_CHUNK_BYTES = 64 * BK * 2;  // one 64(mn) x 64(k) box of an MN-major operand
constexpr int A_SUB_BYTES = BM * BK * 2;     // 16 KB: one CTA's 128 rows of one sub-tile of A

constexpr int MODE_SINGLE = 0, MODE_PAIR = 1, MODE_WIDE = 2;

template <int MODE>
struct Cfg {
    static constexpr bool PAIR = MODE != MODE_SINGLE;
    static constexpr int MSUB = MODE == MODE_WIDE ? 2 : 1;  // 256-row sub-tiles (accumulators) per tile
    static constexpr int ACCS = MODE == MODE_WIDE ? 1 : 2;  // tiles whose accumulators fit in TMEM
    static constexpr int TILE_M = MODE == MODE_SINGLE ? 128 : 256 * MSUB;
    static constexpr int B_ROWS = PAIR ? 128 : 256;  // rows of B staged by one CTA
    static constexpr int A_STAGE_BYTES = MSUB * A_SUB_BYTES;
    static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int STAGES = MODE == MODE_PAIR ? 6 : 4;  // 192 KB of operand stages in every variant
};

// The push epilogue (GEMM -> reduce_scatter) stages 32 rows x 64 columns per epilogue warp in
// shared memory so that what crosses NVLink are whole 128-byte row segments instead of one
// 16-byte piece per lane.  The 16-byte pieces of row r sit at piece index ^ (r & 7), which keeps
// both the per-row writes and the per-segment reads free of bank conflicts without padding.
constexpr int PUSH_WARP_BYTES = 32 * 128;
constexpr int PUSH_STAGING_BYTES = 8 * PUSH_WARP_BYTES;  // up to eight epilogue warps

// The other epilogues leave through TMA stores from 2 KB staging boxes: 16 boxes, two per warp
// in the wide variant (eight epilogue warps), four per warp otherwise.
constexpr int OUT_STAGING_BYTES = 16 * 2048;

template <int EPI>
constexpr int staging_for() {
    return (EPI == EPI_PUSH || EPI == EPI_STORE_ROWS) ? PUSH_STAGING_BYTES : OUT_STAGING_BYTES;
}
template <int MODE, int EPI>
constexpr int stages_for() {
    return Cfg<MODE>::STAGES;
}
template <int MODE, int EPI>
constexpr int smem_for() {
    return stages_for<MODE, EPI>() * Cfg<MODE>::STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/ +
           staging_for<EPI>();
}

struct KParams {
    int M, N, K;
    int m_blocks, n_blocks, num_tiles;
    int group_m;
    int m_rot;
    int n_tile_stride;  // 256, or 128 for the SwiGLU pairing
    int b_half_off;     // row offset of the second 128 rows of a K-major B tile
    __nv_bfloat16* D;
    long ldd;
    __nv_bfloat16* D2;
    long ldd2;
    const __nv_bfloat16* aux;
    long ldaux;
    int aux_off;
    const uint32_t* a_ready;
    int rows_per_flag;
    uint32_t a_ready_target;
    void* const* peer_out;
    int rows_per_peer;
    const int* m_block_group;
    int group_rows_b;
    const int* k_begin;
    const int* k_end;
    int* error_flag;
    int* comm_status;
    uint64_t wait_limit_ns;
    FuseArgs fuse;
};

struct Tile {
    int m0;        // first row of A / D (within the group for grouped-K)
    int n0;        // first output column
    int b_row;     // K-major B: first row; MN-major B: added to the k coordinate
    int k0;        // first k
    int k_blocks;  // 64-wide k steps; 0 = write zeros
    long d_row0;   // first output row
    bool skip;     // nothing to do (padding block of a grouped problem)
};

template <int TILE_M>
__host__ __device__ __forceinline__ Tile decode_tile(const KParams& p, int t) {
    Tile tl;
    tl.skip = false;
    tl.b_row = 0;
    tl.k0 = 0;
    tl.k_blocks = (p.K + BK - 1) / BK;
    int grp = 0;
    if (p.k_begin != nullptr) {  // grouped-K: one dense [M,N] problem per group
        int per = p.m_blocks * p.n_blocks;
        grp = t / per;
        t -= grp * per;
    }
    int per_group = p.group_m * p.n_blocks;
    int g = t / per_group;
    int first_m = g * p.group_m;
    int gsz = p.m_blocks - first_m < p.group_m ? p.m_blocks - first_m : p.group_m;
    int r = t - g * per_group;
    int mb = first_m + r % gsz;
    int nb = r / gsz;
    mb += p.m_rot;
    if (mb >= p.m_blocks)
        mb -= p.m_blocks;
    tl.m0 = mb * TILE_M;
    tl.n0 = nb * p.n_tile_stride;
    tl.d_row0 = tl.m0;
    if (p.k_begin != nullptr) {
        int kb = p.k_begin[grp], ke = p.k_end[grp];
        tl.k0 = kb;
        tl.k_blocks = (ke - kb + BK - 1) / BK;
        tl.d_row0 = static_cast<long>(grp) * p.M + tl.m0;
    } else if (p.m_block_group != nullptr) {
        int e = p.m_block_group[mb];
        if (e < 0)
            tl.skip = true;
        else
            tl.b_row = e * p.group_rows_b;
    }
    return tl;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// 32 consecutive bf16 of one row as 16 packed words; columns from `ncols_ok` on read as zero
__device__ __forceinline__ void load_packed32(const __nv_bfloat16* src, uint32_t (&w)[16], int ncols_ok) {
    if (ncols_ok >= 32) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 q = s4[i];
            w[4 * i] = q.x; w[4 * i + 1] = q.y; w[4 * i + 2] = q.z; w[4 * i + 3] = q.w;
        }
    } else {
        const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t lo16 = 2 * i < ncols_ok ? s16[2 * i] : 0u;
            const uint32_t hi16 = 2 * i + 1 < ncols_ok ? s16[2 * i + 1] : 0u;
            w[i] = lo16 | (hi16 << 16);
        }
    }
}
__device__ __forceinline__ void load_row32(const __nv_bfloat16* src, float (&v)[32], int ncols_ok) {
    if (ncols_ok >= 32) {
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint4 o = s4[i];
            v[i * 8 + 0] = bf16_lo(o.x);
            v[i * 8 + 1] = bf16_hi(o.x);
            v[i * 8 + 2] = bf16_lo(o.y);
            v[i * 8 + 3] = bf16_hi(o.y);
            v[i * 8 + 4] = bf16_lo(o.z);
            v[i * 8 + 5] = bf16_hi(o.z);
            v[i * 8 + 6] = bf16_lo(o.w);
            v[i * 8 + 7] = bf16_hi(o.w);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            v[i] = (i < ncols_ok) ? __bfloat162float(src[i]) : 0.f;
    }
}


// ---------------------------------------------------------------- cluster helpers
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of `addr` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
// TMA load issued by one CTA of a pair; its bytes complete on `bar` (a shared::cluster
// address, here the leader CTA's barrier).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const void* map, uint32_t bar, int c0,
                                                 int c1) {
    asm volatile(
            "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
            " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
            "l"(map), "r"(bar), "r"(c0), "r"(c1)
            : "memory");
}
__device__ __forceinline__ void umma_commit_cg2(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                         bar)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
                 : "memory");
}

// Bounded poll of a flag word until it reaches `target` (wrap-safe).  Warp-uniform result.
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t target, uint64_t limit_ns,
                                              volatile int* abort_flag) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (static_cast<int32_t>(ld_acquire_sys(flag) - target) < 0) {
        poll_pause(spins < 16 ? 64 : 512);
        if ((++spins & 63) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            if (*abort_flag || now - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

// ---------------------------------------------------------------- epilogue of one tile
// `t_addr`: TMEM address of this warp's lane quarter of the accumulator; `row_base`: the first
// of the warp's 32 rows inside the tile.  TMEM loads run one chunk ahead of the arithmetic and
// the stores (two register sets in turn), so their latency is hidden behind the previous chunk.
// 32 fp32 values of one row -> four 16-byte pieces `first`..`first+3` of its 128-byte staging
// row, each stored at piece index ^ sw.
__device__ __forceinline__ void pack_row32_swz(const uint32_t (&r)[32], uint8_t* row, int first, int sw) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint4 o;
        o.x = pack_bf16x2(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
        o.y = pack_bf16x2(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
        o.z = pack_bf16x2(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
        o.w = pack_bf16x2(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
        *reinterpret_cast<uint4*>(row + (((first + i) ^ sw) << 4)) = o;
    }
}

// One epilogue warp's way out to global memory for the TMA-store epilogues: a ring of 2 KB
// staging boxes (32 rows x 32 bf16, 64-byte swizzle) and the output tensor maps.  Lane 0 issues
// every store of the warp, so its bulk groups count them.
struct OutRing {
    uint8_t* base;
    int nslots;  // 2 or 4
    int slot;
    const CUtensorMap* map_d;   // D, columns [0, N)
    const CUtensorMap* map_du;  // D + aux_off, columns [0, N): the second half of a gate/up pair
    const CUtensorMap* map_d2;  // D2
};
constexpr int OUT_BOX_BYTES = 32 * 32 * 2;

// Stores the warp's 32 rows x 32 columns (lane = row, 16 packed pairs) at (row, col) of `map`;
// the tensor map clips what lies past the matrix.
__device__ __forceinline__ void emit_box32(const CUtensorMap* map, OutRing& ring, int lane, int col, int row,
                                           const uint32_t (&pk)[16]) {
    // the store that last used this box has read it
    if (lane == 0) {
        if (ring.nslots == 2)
            tma_store_wait_read<1>();
        else
            tma_store_wait_read<3>();
    }
    __syncwarp();
    uint8_t* buf = ring.base + ring.slot * OUT_BOX_BYTES;
    const int sw = (lane >> 1) & 3;  // 64-byte swizzle: 16-byte piece index ^ address bits 7..8
#pragma unroll
    for (int j = 0; j < 4; ++j)
        *reinterpret_cast<uint4*>(buf + lane * 64 + ((j ^ sw) << 4)) =
                make_uint4(pk[4 * j], pk[4 * j + 1], pk[4 * j + 2], pk[4 * j + 3]);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        tma_store_2d(map, smem_u32(buf), col, row);
        tma_store_commit();
    }
    ring.slot = ring.slot + 1 == ring.nslots ? 0 : ring.slot + 1;
}

template <int EPI>
__device__ __forceinline__ void epilogue_tile(const KParams& p, const Tile& tl, uint32_t t_addr,
                                              int row_base, int lane, bool zero_tile, uint8_t* stage_warp,
                                              OutRing& out, volatile int* abort_flag) {
    const int row_in_tile = row_base + lane;
    if (EPI == EPI_PUSH || EPI == EPI_STORE_ROWS) {
        // The 32 rows of this warp all belong to one owner rank (owners hold whole row blocks).
        // (rows past M are never stored; keep their owner index inside the table)
        const long drow0 = tl.d_row0 + row_base;
        const int peer = EPI == EPI_PUSH ? min(static_cast<int>(drow0 / p.rows_per_peer), 7) : 0;
        const long prow0 = EPI == EPI_PUSH ? drow0 - static_cast<long>(peer) * p.rows_per_peer : drow0;
        __nv_bfloat16* base =
                EPI == EPI_PUSH ? static_cast<__nv_bfloat16*>(p.peer_out != nullptr ? p.peer_out[peer]
                                                                                   : p.fuse.rs_peer_out[peer])
                                : p.D;
        // GEMM -> reduce_scatter: rows this rank owns are not pushed anywhere.  Their tiles come
        // last in every rank's order, so by now the other ranks' partial tiles for these 32 rows x
        // 256 columns have (nearly always) landed in the local staging slots: wait for their
        // counter, then sum the partials in rank order, with this rank's own partial taken from
        // the staging rows in shared memory, and write the output shard.
        const bool own = EPI == EPI_PUSH && p.fuse.rs_out != nullptr && peer == p.fuse.rank;
        if (own && tl.m0 + row_base < p.M) {
            int ok = 1;
            if (lane == 0) {
                const uint32_t* cnt = p.fuse.rs_count_local +
                                      static_cast<size_t>(prow0 / 32) * p.fuse.rs_col_tiles + tl.n0 / BN;
                ok = wait_flag_sys(cnt, p.fuse.rs_target, p.wait_limit_ns, abort_flag) ? 1 : 0;
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok)
                return;  // the wait ran out: the kernel is winding down, nothing more is written
        }
        uint32_t ra[32], rb[32];
        if (zero_tile) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                ra[i] = rb[i] = 0u;
        } else {
            tmem_ld_32x32b_x32(t_addr, ra);
        }
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
            // lane = row: 64 bf16 of this row into its staging row, pieces swizzled by the row
            uint8_t* srow = stage_warp + lane * 128;
            if (!zero_tile) {
                tmem_ld_wait(ra);
                tmem_ld_32x32b_x32(t_addr + c * 64 + 32, rb);
            }
            pack_row32_swz(ra, srow, 0, lane & 7);
            if (!zero_tile) {
                tmem_ld_wait(rb);
                if (c + 1 < BN / 64)
                    tmem_ld_32x32b_x32(t_addr + (c + 1) * 64, ra);
            }
            pack_row32_swz(rb, srow, 4, lane & 7);
            __syncwarp();
            // 8 lanes write one row's 128 bytes: four rows per store instruction
            const int col = tl.n0 + c * 64 + (lane & 7) * 8;
            if (!own) {
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int rr = it * 4 + (lane >> 3);
                    const uint4 v = *reinterpret_cast<const uint4*>(stage_warp + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                    if (tl.m0 + row_base + rr < p.M && col + 8 <= p.N)
                        *reinterpret_cast<uint4*>(base + (prow0 + rr) * p.ldd + col) = v;
                }
            } else {
                const FuseArgs& f = p.fuse;
                const size_t slot_elems = static_cast<size_t>(f.shard_rows) * (f.row_bytes / 2);
                const __nv_bfloat16* slots = static_cast<const __nv_bfloat16*>(f.rs_stage_local);
                const __nv_bfloat16* resid = static_cast<const __nv_bfloat16*>(f.rs_residual);
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(f.rs_out);
                auto add8 = [](float (&acc)[8], const uint4& v) {
                    acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
                    acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
                };
                // two row groups at a time: all partials' loads are issued before the first use
#pragma unroll
                for (int it0 = 0; it0 < 8; it0 += 2) {
                    uint4 part[2][8];
                    uint4 res[2];
                    bool okr[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int rr = (it0 + u) * 4 + (lane >> 3);
                        okr[u] = tl.m0 + row_base + rr < p.M && col + 8 <= p.N;
                        const size_t off = static_cast<size_t>(prow0 + rr) * p.ldd + col;
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (q < f.nranks && q != f.rank && okr[u])
                                part[u][q] = __ldcg(reinterpret_cast<const uint4*>(slots + q * slot_elems + off));
                        if (resid != nullptr && okr[u])
                            res[u] = *reinterpret_cast<const uint4*>(resid + off);
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int rr = (it0 + u) * 4 + (lane >> 3);
                        if (!okr[u])
                            continue;
                        const uint4 mine =
                                *reinterpret_cast<const uint4*>(stage_warp + rr * 128 + (((lane & 7) ^ (rr & 7)) << 4));
                        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            if (q < f.nranks)
                                add8(acc, q == f.rank ? mine : part[u][q]);
                        if (resid != nullptr)
                            add8(acc, res[u]);
                        uint4 o;
                        o.x = pack_bf16x2(acc[0], acc[1]);
                        o.y = pack_bf16x2(acc[2], acc[3]);
                        o.z = pack_bf16x2(acc[4], acc[5]);
                        o.w = pack_bf16x2(acc[6], acc[7]);
                        *reinterpret_cast<uint4*>(dst + static_cast<size_t>(prow0 + rr) * p.ldd + col) = o;
                    }
                }
            }
            __syncwarp();
        }
        return;
    }
    // ---- TMA-store epilogues: 32-column boxes through the warp's ring of staging boxes
    const int m = tl.m0 + row_in_tile;
    const bool row_ok = m < p.M;
    const long drow = tl.d_row0 + row_in_tile;
    const bool rows_in = tl.m0 + row_base < p.M;  // warp-uniform: some of the 32 rows exist
    const int box_row = static_cast<int>(tl.d_row0 + row_base);
    if (EPI == EPI_SWIGLU) {
        // columns [0,128) = gate, [128,256) = up of output columns n0..n0+127
        uint32_t rg[32], ru[32];
        tmem_ld_32x32b_x32(t_addr, rg);
        tmem_ld_32x32b_x32(t_addr + 128, ru);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
            tmem_ld_wait(rg);
            tmem_ld_wait(ru);
            uint32_t pg[16], pu[16], ph[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float g0 = __uint_as_float(rg[2 * i]), g1 = __uint_as_float(rg[2 * i + 1]);
                const float u0 = __uint_as_float(ru[2 * i]), u1 = __uint_as_float(ru[2 * i + 1]);
                pg[i] = pack_bf16x2(g0, g1);
                pu[i] = pack_bf16x2(u0, u1);
                ph[i] = pack_bf16x2(__fdividef(g0, 1.f + __expf(-g0)) * u0,
                                    __fdividef(g1, 1.f + __expf(-g1)) * u1);
            }
            if (c + 1 < 4) {
                tmem_ld_32x32b_x32(t_addr + (c + 1) * 32, rg);
                tmem_ld_32x32b_x32(t_addr + 128 + (c + 1) * 32, ru);
            }
            const int col = tl.n0 + c * 32;
            if (rows_in && col < p.N) {
                emit_box32(out.map_d, out, lane, col, box_row, pg);
                emit_box32(out.map_du, out, lane, col, box_row, pu);
                emit_box32(out.map_d2, out, lane, col, box_row, ph);
            }
        }
        return;
    }
    uint32_t r[32];
    if (zero_tile) {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            r[i] = 0u;
    } else {
        tmem_ld_32x32b_x32(t_addr, r);
    }
    uint4 next_g[4], next_u[4];  // EPI_DSWIGLU: the next chunk's saved gate / up values, packed
    bool have_next = false;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
        const int col = tl.n0 + c * 32;
        const int ok = p.N - col;
        const bool lane_ok = row_ok && ok > 0;
        uint32_t pk[16], pk2[16];
        if (EPI == EPI_STORE_F32) {
            // the accumulator's own bits: two boxes of 16 float columns per 32-column chunk
            if (!zero_tile)
                tmem_ld_wait(r);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                pk[i] = lane_ok || row_ok ? r[i] : 0u;
                pk2[i] = lane_ok || row_ok ? r[16 + i] : 0u;
            }
        } else if (EPI == EPI_STORE) {
            if (!zero_tile)
                tmem_ld_wait(r);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                pk[i] = pack_bf16x2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        } else if (EPI == EPI_ACCUM) {
            float o[32];
            if (lane_ok)
                load_row32(p.D + drow * p.ldd + col, o, ok);
            if (!zero_tile)
                tmem_ld_wait(r);
#pragma unroll
            for (int i = 0; i < 16; ++i)
                pk[i] = lane_ok ? pack_bf16x2(__uint_as_float(r[2 * i]) + o[2 * i],
                                              __uint_as_float(r[2 * i + 1]) + o[2 * i + 1])
                                : 0u;
        } else if (EPI == EPI_DSWIGLU) {
            // saved gate / up values of this chunk, packed (two bf16 per word)
            uint32_t cg[16], cu[16];
            if (lane_ok) {
                if (have_next) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        cg[4 * i] = next_g[i].x; cg[4 * i + 1] = next_g[i].y; cg[4 * i + 2] = next_g[i].z; cg[4 * i + 3] = next_g[i].w;
                        cu[4 * i] = next_u[i].x; cu[4 * i + 1] = next_u[i].y; cu[4 * i + 2] = next_u[i].z; cu[4 * i + 3] = next_u[i].w;
                    }
                } else {
                    load_packed32(p.aux + drow * p.ldaux + col, cg, ok);
                    load_packed32(p.aux + drow * p.ldaux + p.aux_off + col, cu, ok);
                }
            }
            // the saved [G | U] of the next chunk are fetched while this one is worked on
            have_next = false;
            if (row_ok && c + 1 < BN / 32 && ok - 32 >= 32) {
                const uint4* ng = reinterpret_cast<const uint4*>(p.aux + drow * p.ldaux + col + 32);
                const uint4* nu = reinterpret_cast<const uint4*>(p.aux + drow * p.ldaux + p.aux_off + col + 32);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    next_g[i] = __ldg(ng + i);
                    next_u[i] = __ldg(nu + i);
                }
                have_next = true;
            }
            if (!zero_tile)
                tmem_ld_wait(r);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                float dgv[2], duv[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float g = h ? bf16_hi(cg[i]) : bf16_lo(cg[i]);
                    const float u = h ? bf16_hi(cu[i]) : bf16_lo(cu[i]);
                    const float sg = __fdividef(1.f, 1.f + __expf(-g));
                    const float dh = __uint_as_float(r[2 * i + h]);
                    const float silu = g * sg;
                    dgv[h] = dh * u * (sg + silu * (1.f - sg));  // dG
                    duv[h] = dh * silu;                           // dU
                }
                pk[i] = lane_ok ? pack_bf16x2(dgv[0], dgv[1]) : 0u;
                pk2[i] = lane_ok ? pack_bf16x2(duv[0], duv[1]) : 0u;
            }
        }
        if (!zero_tile && c + 1 < BN / 32)
            tmem_ld_32x32b_x32(t_addr + (c + 1) * 32, r);
        if (rows_in && ok > 0) {
            emit_box32(out.map_d, out, lane, col, box_row, pk);
            if (EPI == EPI_DSWIGLU)
                emit_box32(out.map_du, out, lane, col, box_row, pk2);
            if (EPI == EPI_STORE_F32 && ok > 16)
                emit_box32(out.map_d, out, lane, col + 16, box_row, pk2);
        }
    }
}


// ---------------------------------------------------------------- fused all_gather (warps 6..9)
// The communication warps of all CTAs together copy every peer's shard of A into the local
// gather buffer, one shard after the other starting with rank+1, and publish a per-shard
// epoch in `ready` when the last CTA has finished its part.  The TMA producer of the same
// kernel waits for that epoch before it loads rows of the shard.
__device__ __forceinline__ void comm_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__device__ __forceinline__ void copy16(char* dst, const char* src, uint64_t nbytes, int tid) {
    // nbytes is a multiple of 16; both pointers are 16-byte aligned
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
    const uint64_t n = nbytes / 16;
    uint64_t i = tid;
    for (; i + 3ull * COMM_THREADS < n; i += 4ull * COMM_THREADS) {
        const uint4 a = __ldcg(s4 + i), b = __ldcg(s4 + i + COMM_THREADS),
                    c = __ldcg(s4 + i + 2ull * COMM_THREADS), d = __ldcg(s4 + i + 3ull * COMM_THREADS);
        d4[i] = a;
        d4[i + COMM_THREADS] = b;
        d4[i + 2ull * COMM_THREADS] = c;
        d4[i + 3ull * COMM_THREADS] = d;
    }
    for (; i < n; i += COMM_THREADS)
        d4[i] = __ldcg(s4 + i);
}

__device__ __forceinline__ void all_gather_warps(const FuseArgs& f, uint64_t limit_ns,
                                                 volatile int* abort_flag, volatile int* comm_ok) {
    const int tid = threadIdx.x - (NUM_THREADS - COMM_THREADS);
    const int n = f.nranks, rank = f.rank;
    // tell every peer that this rank's shard can be read (earlier kernels of this stream
    // have completed, so the shard is final)
    if (blockIdx.x == 0 && tid < n)
        st_release_sys(f.ag_start_peer[tid] + rank, f.epoch);
    const uint64_t shard_bytes = static_cast<uint64_t>(f.shard_rows) * f.row_bytes;
    const uint64_t per_cta = ((shard_bytes + gridDim.x - 1) / gridDim.x + 15) / 16 * 16;
    const uint64_t b = min(shard_bytes, per_cta * blockIdx.x), e = min(shard_bytes, b + per_cta);
    for (int qq = 0; qq < n; ++qq) {
        const int q = (rank + qq) % n;  // own shard first (local), then rank+1, ...
        const char* src = static_cast<const char*>(f.ag_src[q]);
        char* dst = static_cast<char*>(f.ag_dst) + static_cast<uint64_t>(q) * shard_bytes;
        if (q != rank) {
            // the peer's shard must be final before it is read
            if (tid == 0)
                *comm_ok = wait_flag_sys(f.ag_start_local + q, f.epoch, limit_ns, abort_flag) ? 1 : 0;
            comm_bar();
            const bool ok = *comm_ok != 0;
            comm_bar();
            if (!ok)
                return;  // a wait ran out: the consumer's own bounded wait ends the kernel
        }
        if (src != nullptr && src != dst && e > b)
            copy16(dst + b, src + b, e - b, tid);
        comm_bar();
        if (tid == 0) {
            __threadfence();
            const uint32_t done = atomicAdd(f.ag_count + q, 1u);
            if (done == gridDim.x - 1) {  // the last CTA publishes the shard
                f.ag_count[q] = 0;
                __threadfence();
                st_release_gpu(f.ag_ready + q, f.epoch);
            }
        }
    }
}

template <int MODE, bool A_MN, bool B_MN, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
        gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                         const __grid_constant__ CUtensorMap tma_d, const __grid_constant__ CUtensorMap tma_du,
                         const __grid_constant__ CUtensorMap tma_d2, const KParams p) {
    using C = Cfg<MODE>;
    constexpr bool PAIR = C::PAIR;
    constexpr int MSUB = C::MSUB;
    constexpr int A_STAGE_BYTES = C::A_STAGE_BYTES;
    constexpr int STAGES = stages_for<MODE, EPI>();
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                               ~static_cast<uintptr_t>(1023));
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + STAGES * A_STAGE_BYTES;
    uint8_t* push_staging = smem + STAGES * C::STAGE_BYTES;  // 1024-byte aligned: the staging boxes
    uint64_t* bars = reinterpret_cast<uint64_t*>(push_staging + staging_for<EPI>());
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty.
    // single / pair: tmem_full[a] and tmem_empty[a] belong to accumulator buffer a.
    // wide: tmem_full[0] covers the whole tile, tmem_empty[s] belongs to sub-tile s.
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* comm_ok = reinterpret_cast<volatile int*>(tmem_slot + 2);
    // hand-over of sub-tile 1 to the late-joining second epilogue group (wide variant fused with
    // an all_gather): see the epilogue role below
    int* split_state = reinterpret_cast<int*>(tmem_slot + 3);
    volatile int* g0_tiles = reinterpret_cast<volatile int*>(tmem_slot + 4);  // [4], one per lane quarter

    const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
    const int lane = threadIdx.x & 31;
    // position inside the CTA pair (0 = leader, issues the MMAs); a single CTA is its own leader
    const uint32_t crank = PAIR ? cluster_ctarank() : 0u;
    const int worker = PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
    const int workers = PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);

    const uint32_t full0 = smem_u32(bars);
    const uint32_t empty0 = smem_u32(bars + STAGES);
    const uint32_t tfull0 = smem_u32(bars + 2 * STAGES);
    const uint32_t tempty0 = smem_u32(bars + 2 * STAGES + 2);

    if (threadIdx.x == 0) {
        *abort_flag = 0;
        *split_state = 0;
        for (int i = 0; i < 4; ++i)
            g0_tiles[i] = 0;
        prefetch_tensormap(&tma_a);
        prefetch_tensormap(&tma_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tfull0 + 8 * a, 1);
            // the leader's MMA thread waits for the epilogue warps of both CTAs
            mbar_init(tempty0 + 8 * a, PAIR ? 8 : 4);
        }
        mbar_fence_init();
        fence_proxy_async_smem();
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_cg2(smem_u32(tmem_slot), TMEM_COLS);
            tmem_relinquish_cg2();
        } else {
            tmem_alloc_cg1(smem_u32(tmem_slot), TMEM_COLS);
            tmem_relinquish_cg1();
        }
    }
    tc_fence_before();
    if (PAIR)
        cluster_sync_all();  // barriers of both CTAs exist before any remote arrive / TMA signal
    else
        __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    WaitCtx wc{abort_flag, p.wait_limit_ns};

    if (warp == 0) {
        // ------------------------------------------------------ TMA producer (every CTA)
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool alive = true;
            for (int t = worker; t < p.num_tiles && alive; t += workers) {
                Tile tl = decode_tile<C::TILE_M>(p, t);
                if (tl.skip || tl.k_blocks == 0)
                    continue;
                // this CTA's rows of A: 128 of each 256-row sub-tile
                const int m0 = tl.m0 + static_cast<int>(crank) * BM;
                if (p.a_ready != nullptr) {
                    // all_gather fusion: rows of this m-block arrive from another GPU;
                    // wait (bounded) for the ready counter of each sub-tile's shard.
                    for (int sub = 0; sub < MSUB && alive; ++sub) {
                        if (m0 + sub * 256 >= p.M)
                            break;
                        const uint32_t* f = p.a_ready + (m0 + sub * 256) / p.rows_per_flag;
                        uint32_t spins = 0;
                        uint64_t t0 = 0;
                        while (static_cast<int32_t>(ld_acquire_gpu(f) - p.a_ready_target) < 0) {
                            poll_pause(spins < 16 ? 64 : 256);
                            if ((++spins & 0x3f) == 0) {
                                uint64_t now = globaltimer_ns();
                                if (t0 == 0)
                                    t0 = now;
                                if (*abort_flag || now - t0 > p.wait_limit_ns) {
                                    *abort_flag = 1;
                                    alive = false;
                                    break;
                                }
                            }
                        }
                    }
                    if (!alive)
                        break;
                    fence_proxy_async();  // data written by generic-proxy stores, read by TMA
                }
                for (int kb = 0; kb < tl.k_blocks; ++kb) {
                    if (!mbar_wait(empty0 + 8 * s, ph ^ 1, wc)) {
                        alive = false;
                        break;
                    }
                    const int k = tl.k0 + kb * BK;
                    const uint32_t sa = smem_u32(smem_a + s * A_STAGE_BYTES);
                    const uint32_t sb = smem_u32(smem_b + s * C::B_STAGE_BYTES);
                    if (!PAIR) {
                        const uint32_t fb = full0 + 8 * s;
                        mbar_expect_tx(fb, C::STAGE_BYTES);
                        if (!A_MN) {
                            tma_load_2d(sa, &tma_a, fb, k, m0);
                        } else {
#pragma unroll
                            for (int j = 0; j < BM / 64; ++j)
                                tma_load_2d(sa + j * MN_CHUNK_BYTES, &tma_a, fb, m0 + 64 * j, k);
                        }
                        if (!B_MN) {
                            tma_load_2d(sb, &tma_b, fb, k, tl.b_row + tl.n0);
                            tma_load_2d(sb + C::B_STAGE_BYTES / 2, &tma_b, fb, k,
                                        tl.b_row + tl.n0 + p.b_half_off);
                        } else {
#pragma unroll
                            for (int j = 0; j < C::B_ROWS / 64; ++j)
                                tma_load_2d(sb + j * MN_CHUNK_BYTES, &tma_b, fb, tl.n0 + 64 * j,
                                            tl.b_row + k);
                        }
                    } else {
                        // both CTAs' bytes complete on the leader's barrier
                        const uint32_t fb = mapa_u32(full0 + 8 * s, 0);
                        if (crank == 0)
                            mbar_expect_tx(full0 + 8 * s, 2 * C::STAGE_BYTES);
#pragma unroll
                        for (int sub = 0; sub < MSUB; ++sub) {
                            const uint32_t sas = sa + sub * A_SUB_BYTES;
                            const int ms = m0 + sub * 256;
                            if (!A_MN) {
                                tma_load_2d_pair(sas, &tma_a, fb, k, ms);
                            } else {
#pragma unroll
                                for (int j = 0; j < BM / 64; ++j)
                                    tma_load_2d_pair(sas + j * MN_CHUNK_BYTES, &tma_a, fb, ms + 64 * j, k);
                            }
                        }
                        // this CTA's half of the 256 columns of B
                        if (!B_MN) {
                            tma_load_2d_pair(sb, &tma_b, fb, k,
                                             tl.b_row + tl.n0 + static_cast<int>(crank) * p.b_half_off);
                        } else {
                            const int n0 = tl.n0 + static_cast<int>(crank) * C::B_ROWS;
#pragma unroll
                            for (int j = 0; j < C::B_ROWS / 64; ++j)
                                tma_load_2d_pair(sb + j * MN_CHUNK_BYTES, &tma_b, fb, n0 + 64 * j,
                                                 tl.b_row + k);
                        }
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------ UMMA issuer (leader CTA only)
        if (lane == 0 && crank == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16_f32(PAIR ? 256 : 128, BN, A_MN, B_MN);
            int s = 0;
            uint32_t ph = 0;
            int acc = 0;
            uint32_t acc_ph = 0;
            bool alive = true;
            for (int t = worker; t < p.num_tiles && alive; t += workers) {
                Tile tl = decode_tile<C::TILE_M>(p, t);
                if (tl.skip || tl.k_blocks == 0)
                    continue;
                if (MSUB == 1) {
                    if (!mbar_wait<PAIR>(tempty0 + 8 * acc, acc_ph ^ 1, wc))
                        break;
                    tc_fence_after();
                }
                for (int kb = 0; kb < tl.k_blocks; ++kb) {
                    if (!mbar_wait(full0 + 8 * s, ph, wc)) {
                        alive = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sb = smem_u32(smem_b + s * C::B_STAGE_BYTES);
#pragma unroll
                    for (int sub = 0; sub < MSUB; ++sub) {
                        if (MSUB > 1 && kb == 0) {
                            // the epilogue of the previous tile has drained this sub-tile's accumulator
                            if (!mbar_wait<PAIR>(tempty0 + 8 * sub, acc_ph ^ 1, wc)) {
                                alive = false;
                                break;
                            }
                            tc_fence_after();
                        }
                        const uint32_t d_tmem = tmem_base + (MSUB > 1 ? sub : acc) * BN;
                        const uint32_t sa = smem_u32(smem_a + s * A_STAGE_BYTES + sub * A_SUB_BYTES);
#pragma unroll
                        for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                            // K-major: 16 k = 32 bytes inside the 128 B row.
                            // MN-major: 16 k = 16 rows of 128 B.
                            const uint64_t ad =
                                    A_MN ? umma_smem_desc_sw128(sa + kk * (UMMA_K * 128), MN_CHUNK_BYTES,
                                                                1024)
                                         : umma_smem_desc_sw128(sa + kk * (UMMA_K * 2), 16, 1024);
                            const uint64_t bd =
                                    B_MN ? umma_smem_desc_sw128(sb + kk * (UMMA_K * 128), MN_CHUNK_BYTES,
                                                                1024)
                                         : umma_smem_desc_sw128(sb + kk * (UMMA_K * 2), 16, 1024);
                            if (PAIR)
                                umma_f16_cg2(d_tmem, ad, bd, idesc, (kb | kk) != 0 ? 1u : 0u);
                            else
                                umma_f16_cg1(d_tmem, ad, bd, idesc, (kb | kk) != 0 ? 1u : 0u);
                        }
                    }
                    if (!alive)
                        break;
                    // free the smem stage (in both CTAs of a pair) when these MMAs retire
                    if (PAIR) {
                        umma_commit_cg2(empty0 + 8 * s);
                        umma_commit_cg2(mapa_u32(empty0 + 8 * s, 1));
                    } else {
                        umma_commit_cg1(empty0 + 8 * s);
                    }
                    if (++s == STAGES) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!alive)
                    break;
                // accumulator complete: wake the epilogue warps (of both CTAs)
                if (PAIR) {
                    umma_commit_cg2(tfull0 + 8 * acc);
                    umma_commit_cg2(mapa_u32(tfull0 + 8 * acc, 1));
                } else {
                    umma_commit_cg1(tfull0 + 8 * acc);
                }
                if (++acc == C::ACCS) {
                    acc = 0;
                    acc_ph ^= 1;
                }
            }
        }
    } else {
        // ------------------------------------------------------ warps 2..9
        // Warps 2..5 are the epilogue group of every variant.  In the wide variant warps 6..9 are
        // a second epilogue group: the first group drains sub-tile 0 while the second drains
        // sub-tile 1.
        //  * Nothing to gather: both groups start with the first tile and stay within one phase
        //    of the accumulator barrier (the MMA warp needs both sub-tiles drained to go on), so
        //    its parity is enough for both.
        //  * Fused with an all_gather: warps 6..9 gather first and join late, at a tile ordinal S
        //    that nobody can know in advance, and a late joiner cannot tell the barrier's phases
        //    apart by parity.  So (a) S is agreed through one shared word: every first-group warp
        //    records each ordinal it starts with atomicMax before it decides how much of that
        //    tile is its own, and the second group's leader claims S = first ordinal not yet
        //    recorded with a compare-and-swap; whoever saw no claim at ordinal i has made S > i.
        //    (b) From S on, first-group warp q tells second-group warp q through a counter in
        //    shared memory that tile i's accumulators are complete.
        constexpr int DECIDED = 0x40000000;
        const bool second = warp >= 6;
        const bool late_join = MSUB > 1 && p.fuse.ag_dst != nullptr;
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        int split_from = MSUB > 1 ? (late_join ? 0x3fffffff : 0) : 0x3fffffff;
        if (second && p.fuse.ag_dst != nullptr) {
            all_gather_warps(p.fuse, p.wait_limit_ns, abort_flag, comm_ok);
            if (late_join) {
                if (threadIdx.x == NUM_THREADS - COMM_THREADS) {
                    int cur = *reinterpret_cast<volatile int*>(split_state);
                    for (;;) {
                        const int old = atomicCAS(split_state, cur, DECIDED | cur);
                        if (old == cur)
                            break;
                        cur = old;
                    }
                }
                comm_bar();
                split_from = *reinterpret_cast<volatile int*>(split_state) & ~DECIDED;
            }
        }
        if (!second || MSUB > 1) {
            OutRing out;
            out.nslots = MSUB > 1 ? 2 : 4;
            out.base = push_staging + (MSUB > 1 ? (warp - 2) * 2 : q * 4) * OUT_BOX_BYTES;
            out.slot = 0;
            out.map_d = &tma_d;
            out.map_du = &tma_du;
            out.map_d2 = &tma_d2;
            uint8_t* stage_warp = push_staging + (MSUB > 1 ? warp - 2 : q) * PUSH_WARP_BYTES;
            int acc = 0;
            uint32_t acc_ph = 0;
            int ordinal = 0;
            for (int t = worker; t < p.num_tiles; t += workers) {
                Tile tl = decode_tile<C::TILE_M>(p, t);
                if (tl.skip)
                    continue;
                const bool zero_tile = tl.k_blocks == 0;
                const int i = ordinal++;
                if (late_join && !second) {
                    int old = 0;
                    if (lane == 0)
                        old = atomicMax(split_state, i + 1);
                    old = __shfl_sync(0xffffffffu, old, 0);
                    if (old & DECIDED)
                        split_from = old & ~DECIDED;
                }
                const bool split = i >= split_from;
                const int sub_begin = second ? 1 : 0;
                const int sub_end = second ? (split ? 2 : 1) : (split ? 1 : MSUB);
                if (!zero_tile && sub_begin < sub_end) {
                    // the whole warp must agree before the .sync.aligned TMEM loads
                    bool got;
                    if (late_join && second) {
                        // first-group warp q has seen the accumulator barrier of tile i complete
                        got = true;
                        uint32_t spins = 0;
                        uint64_t t0 = 0;
                        while (g0_tiles[q] < i + 1) {
                            poll_pause(128);
                            if ((++spins & 0x3f) == 0) {
                                const uint64_t now = globaltimer_ns();
                                if (t0 == 0)
                                    t0 = now;
                                if (*abort_flag || now - t0 > p.wait_limit_ns) {
                                    *abort_flag = 1;
                                    got = false;
                                    break;
                                }
                            }
                        }
                    } else {
                        // one lane sleeps on the barrier for the warp
                        got = lane == 0 ? mbar_wait(tfull0 + 8 * acc, acc_ph, wc) : true;
                    }
                    if (!__all_sync(0xffffffffu, got))
                        break;
                    tc_fence_after();
                    if (late_join && !second) {
                        tc_fence_before();
                        if (lane == 0)
                            g0_tiles[q] = i + 1;
                    }
                }
#pragma unroll 1
                for (int sub = sub_begin; sub < sub_end; ++sub) {
                    const int sub_row = sub * 256 + static_cast<int>(crank) * BM;  // this CTA's rows of the sub-tile
                    const uint32_t t_addr =
                            tmem_base + (MSUB > 1 ? sub : acc) * BN + (static_cast<uint32_t>(q * 32) << 16);
                    epilogue_tile<EPI>(p, tl, t_addr, sub_row + q * 32, lane, zero_tile, stage_warp, out, abort_flag);
                    if (!zero_tile) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            const uint32_t eb = tempty0 + 8 * (MSUB > 1 ? sub : acc);
                            if (PAIR && crank != 0)
                                mbar_arrive_remote(mapa_u32(eb, 0));
                            else
                                mbar_arrive(eb);
                        }
                    }
                    if (EPI == EPI_PUSH && p.fuse.rs_count_peer[0] != nullptr && tl.m0 + sub_row < p.M) {
                        // this warp's 32 rows x 256 columns of the partial tile are in the owner's
                        // staging slot: make them visible system-wide, then count them in the
                        // owner's counter of that (row group, column tile)
                        __syncwarp();
                        const int row0 = tl.m0 + sub_row + q * 32;
                        const int owner = row0 / p.rows_per_peer;
                        if (lane == 0 && owner != p.fuse.rank) {
                            const size_t idx = static_cast<size_t>((row0 - owner * p.rows_per_peer) / 32) *
                                                       p.fuse.rs_col_tiles + tl.n0 / BN;
                            __threadfence_system();
                            red_release_sys_add(p.fuse.rs_count_peer[owner] + idx, 1u);
                        }
                    }
                }
                if (!zero_tile) {
                    if (++acc == C::ACCS) {
                        acc = 0;
                        acc_ph ^= 1;
                    }
                }
            }
            // this thread's TMA stores have left shared memory before the CTA gives it up
            if (lane == 0)
                tma_store_wait<0>();
        }
    }
    // ---------------------------------------------------------- teardown
    __syncwarp();
    tc_fence_before();
    if (PAIR)
        cluster_sync_all();  // the peer may still read this CTA's smem / signal its barriers
    else
        __syncthreads();
    if (*abort_flag) {
        // A wait ran out.  TMA copies already issued complete on their own within
        // microseconds (their source is local memory); give them that time before
        // shared memory is released, then report.
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000) {
        }
        if (threadIdx.x == 0 && p.error_flag != nullptr)
            atomicExch(p.error_flag, 1);
        // a fused collective's wait ran out: the communicator learns of it as MEGRAY_TIMEOUT
        if (threadIdx.x == 0 && p.comm_status != nullptr)
            atomicCAS(p.comm_status, 0, 12);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR)
            tmem_dealloc_cg2(tmem_base, TMEM_COLS);
        else
            tmem_dealloc_cg1(tmem_base, TMEM_COLS);
    }
}

// ------------------------------------------------------------------ host side

PFN_cuTensorMapEncodeTiled_v12000 get_encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) ==
                    cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(f);
    });
    return fn;
}

// bf16 matrix, `inner` contiguous elements per row, `outer` rows `ld` elements apart;
// box = 64 inner elements (128 B, the swizzle span) x `box_rows`.
bool make_map(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint64_t ld,
              uint32_t box_rows) {
    auto fn = get_encode_fn();
    if (fn == nullptr)
        return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Output matrix for the TMA-store epilogues: box = 32 columns (64 B, the swizzle span) x 32 rows;
// for a float32 matrix 16 columns x 32 rows (the same 64-byte rows).
bool make_out_map(CUtensorMap* map, const void* ptr, uint64_t cols, uint64_t rows, uint64_t ld, bool f32 = false) {
    auto fn = get_encode_fn();
    if (fn == nullptr)
        return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * (f32 ? 4u : 2u)};
    cuuint32_t box[2] = {f32 ? 16u : 32u, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

struct Maps {
    CUtensorMap a, b, d, du, d2;
};

std::atomic<uint64_t> g_launches{0};

// Launches one instantiation.  `workers` = CTAs (single) or CTA pairs (pair) wanted at most;
// the pair variant is additionally capped by what the device can co-schedule as 2-CTA clusters.
template <int MODE, bool A_MN, bool B_MN, int EPI>
cudaError_t launch_t(const Maps& maps, const KParams& kp, int workers, cudaStream_t stream) {
    constexpr bool PAIR = Cfg<MODE>::PAIR;
    auto kern = gemm_bf16_kernel<MODE, A_MN, B_MN, EPI>;
    constexpr int smem = smem_for<MODE, EPI>();
    int dev = 0;
    cudaGetDevice(&dev);
    static std::mutex mu;
    static std::map<int, int> max_workers;  // per device: attribute set, cluster capacity known
    int cap = 0;
    {
        std::lock_guard<std::mutex> lk(mu);
        auto it = max_workers.find(dev);
        if (it == max_workers.end()) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            if (e != cudaSuccess)
                return e;
            int n = 0;
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
            if (PAIR) {
                cudaLaunchConfig_t qc = {};
                qc.gridDim = dim3(static_cast<unsigned>(n / 2 * 2));
                qc.blockDim = dim3(NUM_THREADS);
                qc.dynamicSmemBytes = smem;
                cudaLaunchAttribute qa[1];
                qa[0].id = cudaLaunchAttributeClusterDimension;
                qa[0].val.clusterDim.x = 2;
                qa[0].val.clusterDim.y = 1;
                qa[0].val.clusterDim.z = 1;
                qc.attrs = qa;
                qc.numAttrs = 1;
                int clusters = 0;
                e = cudaOccupancyMaxActiveClusters(&clusters, kern, &qc);
                if (e != cudaSuccess || clusters <= 0) {
                    (void)cudaGetLastError();
                    clusters = n / 2;
                }
                n = clusters;
            }
            max_workers[dev] = n;
            cap = n;
        } else {
            cap = it->second;
        }
    }
    if (workers > cap)
        workers = cap;
    if (workers < 1)
        workers = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(PAIR ? 2 * workers : workers));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = PAIR ? 2 : 1;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, maps.a, maps.b, maps.d, maps.du, maps.d2, kp);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    count_launch();
    return e;
}

template <int MODE, bool A_MN, bool B_MN>
cudaError_t launch_e(int epi, const Maps& maps, const KParams& kp, int workers, cudaStream_t stream) {
    switch (epi) {
        case EPI_STORE:
            return launch_t<MODE, A_MN, B_MN, EPI_STORE>(maps, kp, workers, stream);
        case EPI_ACCUM:
            return launch_t<MODE, A_MN, B_MN, EPI_ACCUM>(maps, kp, workers, stream);
        case EPI_PUSH:
            return launch_t<MODE, A_MN, B_MN, EPI_PUSH>(maps, kp, workers, stream);
        case EPI_STORE_ROWS:
            return launch_t<MODE, A_MN, B_MN, EPI_STORE_ROWS>(maps, kp, workers, stream);
        case EPI_STORE_F32:
            return launch_t<MODE, A_MN, B_MN, EPI_STORE_F32>(maps, kp, workers, stream);
        case EPI_DSWIGLU:
            return launch_t<MODE, A_MN, B_MN, EPI_DSWIGLU>(maps, kp, workers, stream);
        case EPI_SWIGLU:
            if (B_MN)
                return cudaErrorInvalidValue;
            return launch_t<MODE, A_MN, false, EPI_SWIGLU>(maps, kp, workers, stream);
        default:
            return cudaErrorInvalidValue;
    }
}

template <int MODE>
cudaError_t launch_l(bool a_mn, bool b_mn, int epi, const Maps& maps, const KParams& kp, int workers,
                     cudaStream_t stream) {
    if (!a_mn && !b_mn)
        return launch_e<MODE, false, false>(epi, maps, kp, workers, stream);
    if (!a_mn && b_mn)
        return launch_e<MODE, false, true>(epi, maps, kp, workers, stream);
    if (a_mn && !b_mn)
        return launch_e<MODE, true, false>(epi, maps, kp, workers, stream);
    return launch_e<MODE, true, true>(epi, maps, kp, workers, stream);
}

int sm_count() {
    static std::mutex mu;
    static std::map<int, int> cache;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lk(mu);
    auto it = cache.find(dev);
    if (it != cache.end())
        return it->second;
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cache[dev] = n;
    return n;
}

}  // namespace

uint64_t gemm_launch_count() { return g_launches.load(std::memory_order_relaxed); }

namespace {
// Tile variant and raster of a problem: what launch_gemm_bf16 runs and tile_schedule reports.
struct Plan {
    bool pair, wide;
    int tile_m;
};
Plan plan_tiles(const GemmArgs& a, KParams* kpp, int sms) {
    KParams& kp = *kpp;
    const bool grouped_m = a.grouped.m_block_group != nullptr;
    const bool grouped_k = a.grouped.k_begin != nullptr;
    // A CTA pair per tile unless rows are grouped in 128-row blocks (per-expert
    // forward/backward), which need the 128-row tile.  Large dense problems take the
    // 512-row tile: less operand traffic per FLOP, at the price of an epilogue that is
    // only half hidden, which a long K loop amortises.
    // MEGRAY_GEMM_VARIANT stands in for variant 0 (a tuning and test aid)
    static const int env_variant = [] {
        const char* e = getenv("MEGRAY_GEMM_VARIANT");
        return e != nullptr ? atoi(e) : 0;
    }();
    const int variant = a.variant != 0 ? a.variant : env_variant;
    Plan pl;
    pl.pair = !grouped_m && variant != 1 && a.M > 128;
    pl.wide = pl.pair && variant == 3;
    if (pl.pair && variant == 0 && !grouped_k) {
        const long tiles_wide = static_cast<long>((a.M + 511) / 512) *
                                ((a.N + (a.epilogue == EPI_SWIGLU ? 127 : 255)) / (a.epilogue == EPI_SWIGLU ? 128 : 256));
        // (the dSwiGLU epilogue reads and writes four values per accumulator element; it needs
        // the next tile's main loop to hide behind: 12.9-13.2 ms on the pair tile against
        // 13.3-14.0 ms on the wide one for 32768 x 28672 x 8192)
        pl.wide = a.M >= 1024 && a.K >= 3072 && tiles_wide >= 2L * (sms / 2) && a.epilogue != EPI_DSWIGLU;
    }
    // GEMM -> reduce_scatter waits, in the tiles of the rows it owns, for the other ranks' tiles of
    // the same rows.  That cannot deadlock as long as those tiles come strictly earlier in the
    // other ranks' order, which the row rotation guarantees when a shard is a whole number of tiles.
    if (pl.wide && a.fuse.rs_out != nullptr && a.fuse.shard_rows % 512 != 0)
        pl.wide = false;
    pl.tile_m = pl.wide ? 512 : pl.pair ? 256 : BM;
    const int tile_m = pl.tile_m;
    kp.M = a.M;
    kp.N = a.N;
    kp.K = a.K;
    kp.m_blocks = (a.M + tile_m - 1) / tile_m;
    kp.n_tile_stride = (a.epilogue == EPI_SWIGLU) ? 128 : BN;
    kp.b_half_off = (a.epilogue == EPI_SWIGLU) ? a.aux_off : 128;
    kp.n_blocks = (a.N + kp.n_tile_stride - 1) / kp.n_tile_stride;
    kp.num_tiles = kp.m_blocks * kp.n_blocks * (grouped_k ? a.grouped.groups : 1);
    // concurrently running tiles form a compact patch (2048 rows x 2300 columns for the 128- and
    // 256-row tiles, 4096 x 2300 for the 512-row tile, which measured 2-5 % faster than 2048 x 4700)
    // so that each loaded A / B panel is shared by as many tiles as possible in L2
    kp.group_m = pl.pair ? 8 : 16;
    {
        // tuning aid: MEGRAY_GEMM_GROUP_M overrides the raster's m-blocks per column sweep
        static const int env_group_m = [] {
            const char* e = getenv("MEGRAY_GEMM_GROUP_M");
            return e != nullptr ? atoi(e) : 0;
        }();
        if (env_group_m > 0)
            kp.group_m = env_group_m;
    }
    {
        const int rot_blocks = a.m_rot / tile_m;  // m_rot is given in rows
        kp.m_rot = (rot_blocks % kp.m_blocks + kp.m_blocks) % kp.m_blocks;
    }
    kp.m_block_group = a.grouped.m_block_group;
    kp.group_rows_b = a.grouped.group_rows_b;
    kp.k_begin = a.grouped.k_begin;
    kp.k_end = a.grouped.k_end;
    return pl;
}
}  // namespace

int tile_schedule(const GemmArgs& a, int sms, int* tiles, int max_tiles) {
    if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.grouped.m_block_group != nullptr || a.grouped.k_begin != nullptr)
        return -1;
    KParams kp{};
    const Plan pl = plan_tiles(a, &kp, sms);
    for (int t = 0; t < kp.num_tiles && t < max_tiles; ++t) {
        const Tile tl = pl.wide ? decode_tile<512>(kp, t) : pl.pair ? decode_tile<256>(kp, t) : decode_tile<128>(kp, t);
        tiles[4 * t + 0] = tl.m0;
        tiles[4 * t + 1] = tl.n0;
        tiles[4 * t + 2] = pl.tile_m;
        tiles[4 * t + 3] = kp.n_tile_stride;
    }
    return kp.num_tiles;
}

cudaError_t launch_gemm_bf16(const GemmArgs& a, cudaStream_t stream) {
    if (a.M <= 0 || a.N <= 0 || a.K <= 0)
        return cudaErrorInvalidValue;
    if ((a.lda % 8) || (a.ldb % 8) || (a.ldd % 8))
        return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(a.A) | reinterpret_cast<uintptr_t>(a.B) |
         reinterpret_cast<uintptr_t>(a.D)) & 15)
        return cudaErrorInvalidValue;
    const bool grouped_m = a.grouped.m_block_group != nullptr;
    const bool grouped_k = a.grouped.k_begin != nullptr;
    KParams kp{};
    const Plan pl = plan_tiles(a, &kp, sm_count());
    const bool pair = pl.pair, wide = pl.wide;
    const int tile_m = pl.tile_m;
    kp.D = static_cast<__nv_bfloat16*>(a.D);
    kp.ldd = a.ldd;
    kp.D2 = static_cast<__nv_bfloat16*>(a.D2);
    kp.ldd2 = a.ldd2;
    kp.aux = static_cast<const __nv_bfloat16*>(a.aux);
    kp.ldaux = a.ldaux;
    kp.aux_off = a.aux_off;
    kp.a_ready = a.a_ready;
    kp.rows_per_flag = a.rows_per_flag > 0 ? a.rows_per_flag : BM;
    kp.a_ready_target = a.a_ready_target;
    kp.peer_out = a.peer_out;
    kp.rows_per_peer = a.rows_per_peer > 0 ? a.rows_per_peer : a.M;
    kp.error_flag = a.error_flag;
    kp.comm_status = a.comm_status;
    kp.wait_limit_ns = a.wait_limit_ns ? a.wait_limit_ns : 4000000000ull;
    kp.fuse = a.fuse;

    if (a.epilogue == EPI_SWIGLU && (a.D2 == nullptr || (a.ldd2 % 8)))
        return cudaErrorInvalidValue;
    if (a.epilogue == EPI_DSWIGLU && (a.aux == nullptr || (a.ldaux % 8)))
        return cudaErrorInvalidValue;
    if (a.epilogue == EPI_PUSH &&
        ((a.peer_out == nullptr && a.fuse.rs_peer_out[0] == nullptr) || (kp.rows_per_peer % (pair ? 256 : BM))))
        return cudaErrorInvalidValue;
    if ((a.epilogue == EPI_PUSH || a.epilogue == EPI_STORE_ROWS) && (a.N % 8))
        return cudaErrorInvalidValue;
    if (a.a_ready != nullptr && (kp.rows_per_flag % BM))
        return cudaErrorInvalidValue;

    // Extents the tensor maps cover.  Grouped problems stack the groups along the
    // outer dimension of B.
    const uint64_t groups = (grouped_m || grouped_k) ? static_cast<uint64_t>(a.grouped.groups) : 1;
    Maps maps;
    CUtensorMap& ma = maps.a;
    CUtensorMap& mb = maps.b;
    bool ok;
    if (!a.a_mn) {
        ok = make_map(&ma, a.A, a.K, a.M, a.lda, BM);
    } else {
        // stored [K, M]; for grouped-K, K counts the rows of all groups together
        ok = make_map(&ma, a.A, a.M, a.K, a.lda, BK);
    }
    if (!ok)
        return cudaErrorInvalidValue;
    if (!a.b_mn) {
        // SwiGLU pairing reads rows n and n+aux_off: the map spans both halves.
        uint64_t rows = (a.epilogue == EPI_SWIGLU) ? static_cast<uint64_t>(a.aux_off) + a.N
                                                   : static_cast<uint64_t>(a.N);
        if (grouped_m)
            rows = groups * static_cast<uint64_t>(a.grouped.group_rows_b);
        ok = make_map(&mb, a.B, a.K, rows, a.ldb, 128);
    } else {
        uint64_t krows = static_cast<uint64_t>(a.K);
        if (grouped_m)
            krows = groups * static_cast<uint64_t>(a.grouped.group_rows_b);
        ok = make_map(&mb, a.B, a.N, krows, a.ldb, BK);
    }
    if (!ok)
        return cudaErrorInvalidValue;

    int workers = kp.num_tiles;
    if (a.sm_limit > 0) {
        const int lim = pair ? a.sm_limit / 2 : a.sm_limit;
        if (lim < workers)
            workers = lim > 0 ? lim : 1;
    }
    // Output maps of the TMA-store epilogues.  A grouped-K problem stacks one [M, N] result per
    // group; rows that a tile has past M would land in the next group's result, so such shapes
    // (M not a multiple of the tile) leave through the guarded row-segment stores instead.
    int epi = a.epilogue;
    const uint64_t out_rows = static_cast<uint64_t>(a.M) * (grouped_k ? groups : 1);
    if (epi == EPI_STORE && grouped_k && (a.M % tile_m)) {
        if (a.N % 8)
            return cudaErrorInvalidValue;
        epi = EPI_STORE_ROWS;
    }
    if (epi == EPI_PUSH || epi == EPI_STORE_ROWS) {
        maps.d = maps.du = maps.d2 = maps.a;  // not used by these epilogues
    } else {
        if (grouped_k && (a.M % tile_m))
            return cudaErrorInvalidValue;
        ok = make_out_map(&maps.d, a.D, a.N, out_rows, a.ldd, epi == EPI_STORE_F32);
        maps.du = maps.d2 = maps.d;
        if (ok && (epi == EPI_SWIGLU || epi == EPI_DSWIGLU)) {
            if (a.aux_off % 8)
                return cudaErrorInvalidValue;
            ok = make_out_map(&maps.du, static_cast<const __nv_bfloat16*>(a.D) + a.aux_off, a.N, out_rows, a.ldd);
        }
        if (ok && epi == EPI_SWIGLU)
            ok = make_out_map(&maps.d2, a.D2, a.N, out_rows, a.ldd2);
        if (!ok)
            return cudaErrorInvalidValue;
    }
    if (wide)
        return launch_l<MODE_WIDE>(a.a_mn, a.b_mn, epi, maps, kp, workers, stream);
    if (pair)
        return launch_l<MODE_PAIR>(a.a_mn, a.b_mn, epi, maps, kp, workers, stream);
    return launch_l<MODE_SINGLE>(a.a_mn, a.b_mn, epi, maps, kp, workers, stream);
}

}  // namespace gemm
}  // namespace mgk
