// Host-visible declarations of the tcgen05 bf16 GEMM family.
//
// One persistent, warp-specialised kernel template computes
//     D[M,N] = A[M,K] * B[N,K]^T        (fp32 accumulation in TMEM)
// for bf16 operands that are each either K-major (row-major [rows, K]) or
// MN-major (stored [K, rows]); the epilogue variant decides what is written.
// The reference library has no GEMM: these kernels serve the tensor-parallel
// MLP and the expert-parallel MoE entry points built on the collectives.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace mgk {
namespace gemm {

enum Epilogue : int {
    EPI_STORE = 0,    // D = acc (bf16)
    EPI_SWIGLU = 1,   // acc tile = [gate | up]; writes G,U into D (cols n and n+aux_off) and
                      // silu(G)*U into D2
    EPI_DSWIGLU = 2,  // acc = dH; reads G,U from aux, writes dG,dU into D (cols n, n+aux_off)
    EPI_ACCUM = 3,    // D = acc + D (bf16 read-modify-write; used for gradient accumulation)
    EPI_PUSH = 4,     // D row blocks live on different GPUs: row r goes to peer_out[r / rows_per_peer]
    EPI_STORE_ROWS = 5,  // D = acc, written as whole 128-byte row segments through shared memory
    EPI_STORE_F32 = 6,   // D = acc as float32 (D is a float matrix, ldd in float elements): the partial
                         // products of a K split, which are summed before anything is rounded to bf16
};

// One m-block of a grouped (per-expert) problem.
struct GroupedArgs {
    const int* m_block_group;  // [m_blocks] group (expert) of each 128-row block, -1 = skip
    int group_rows_b;          // rows of B per group (B is [groups*group_rows_b, K], K-major), or
                               // for MN-major B: B is [groups][K, N] and this is K
    const int* k_begin;        // grouped-K (weight gradient): per group first row of the K range
    const int* k_end;          //   and one past the last; null otherwise
    int groups;
};

// Collective fused into the GEMM (all pointers are addresses valid on this GPU; peers'
// memory is reached through the symmetric heap mapping).
struct FuseArgs {
    int nranks, rank;
    int shard_rows;      // rows of one rank's shard of the gathered / scattered matrix
    int row_bytes;       // bytes of one row (rows are contiguous)
    uint32_t epoch;      // this call's value for the start flags and ready words
    // all_gather -> GEMM: the communication warps copy shard q from ag_src[q] into
    // ag_dst + q * shard bytes (own shard: local copy, or nothing when ag_src[rank] is the
    // destination itself) and publish `epoch` in ag_ready[q]; pass ag_ready as `a_ready`.
    void* ag_dst;                    // null = no fused gather
    const void* ag_src[8];
    uint32_t* ag_ready;              // [nranks] local
    uint32_t* ag_count;              // [nranks] local, zero between calls
    uint32_t* ag_start_peer[8];      // peer q's start-flag array (this rank writes slot [rank])
    const uint32_t* ag_start_local;  // this rank's start-flag array [nranks]
    // GEMM -> reduce_scatter (EPI_PUSH): rs_peer_out[p] is rank p's staging slot for this rank's
    // partial rows.  Every finished piece of 32 rows x 256 columns that belongs to another rank
    // bumps that rank's counter [row group of the shard][column tile] (rs_count_peer[p]).  Rows
    // this rank owns are not pushed: their tiles come last in the tile order, and their epilogue
    // waits until the counter of its piece reaches rs_target (all other ranks have delivered),
    // adds the other ranks' staged partials (rs_stage_local, slot q = rank q's rows) and
    // rs_residual to its own partial in rank order and writes rs_out.
    void* rs_peer_out[8];            // rank p's staging slot for this rank's partial rows
    uint32_t* rs_count_peer[8];      // [0] null = no counting
    const uint32_t* rs_count_local;  // [shard_rows / 32][rs_col_tiles]
    int rs_col_tiles;                // 256-column tiles per row: (N + 255) / 256
    uint32_t rs_target;              // (nranks - 1) x (calls on these counters so far, this one included)
    const void* rs_stage_local;      // this rank's n staging slots, slot q = rank q's partial rows
    void* rs_out;                    // null = plain push (no reduction in this kernel)
    const void* rs_residual;         // optional: added to the reduced shard
};

struct GemmArgs {
    const void* A;
    const void* B;
    void* D;
    void* D2;         // EPI_SWIGLU: H output
    const void* aux;  // EPI_DSWIGLU: saved [G | U]
    int M, N, K;
    long lda, ldb, ldd, ldd2, ldaux;  // leading dimensions in elements
    bool a_mn, b_mn;                  // operand is MN-major (stored [K, rows])
    int epilogue;
    int aux_off;  // column offset of the U half (EPI_SWIGLU / EPI_DSWIGLU), also B row offset
    int m_rot;    // start the row-block order at this row (all_gather fused GEMM: own shard first)
    int sm_limit; // 0 = all SMs; otherwise cap on the persistent grid
    int variant;  // 0 = automatic, 1 = single-CTA 128 x 256 tile, 2 = CTA-pair 256 x 256 tile, 3 = CTA-pair 512 x 256 tile
    // all_gather fusion: wait until a_ready[(m_block*128)/rows_per_flag] >= a_ready_target
    const uint32_t* a_ready;
    int rows_per_flag;
    uint32_t a_ready_target;
    // reduce_scatter fusion (EPI_PUSH): per-peer output base pointers, rows per peer
    void* const* peer_out;  // device array [n_peers]
    int rows_per_peer;
    // grouped problems (MoE); null m_block_group = dense
    GroupedArgs grouped;
    FuseArgs fuse;            // zero-initialised = no fused collective
    int* error_flag;          // device word; non-zero after a wait ran out
    int* comm_status;         // optional: a communicator's status word, set to MEGRAY_TIMEOUT then
    uint64_t wait_limit_ns;   // 0 = default (4 s)
};

// Launches on `stream`.  Returns cudaSuccess or the launch / argument error.
// Requirements: bf16 data, base pointers 16-byte aligned, leading dimensions
// multiples of 8 elements, K > 0.
cudaError_t launch_gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// Host-side view of the tile raster of a dense problem on a device with `sms` SMs: writes
// (m0, n0, tile rows, output columns per tile) for each tile in launch order (tile t runs on
// worker t mod workers) into `tiles` (4 ints per tile, at most `max_tiles` tiles) and returns
// the number of tiles, or -1 for grouped problems.  Needs no GPU.
int tile_schedule(const GemmArgs& args, int sms, int* tiles, int max_tiles);

// Number of kernels this module has launched since load (for launch accounting).
uint64_t gemm_launch_count();

}  // namespace gemm
}  // namespace mgk
