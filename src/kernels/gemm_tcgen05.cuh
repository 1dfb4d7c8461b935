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
    int variant;  // 0 = automatic, 1 = force the single-CTA 128 x 256 tile
    // all_gather fusion: wait until a_ready[(m_block*128)/rows_per_flag] >= a_ready_target
    const uint32_t* a_ready;
    int rows_per_flag;
    uint32_t a_ready_target;
    // reduce_scatter fusion (EPI_PUSH): per-peer output base pointers, rows per peer
    void* const* peer_out;  // device array [n_peers]
    int rows_per_peer;
    uint32_t* tile_done;    // optional: counter bumped once per finished tile (gpu scope)
    // grouped problems (MoE); null m_block_group = dense
    GroupedArgs grouped;
    int* error_flag;          // device word; non-zero after a wait ran out
    uint64_t wait_limit_ns;   // 0 = default (4 s)
};

// Launches on `stream`.  Returns cudaSuccess or the launch / argument error.
// Requirements: bf16 data, base pointers 16-byte aligned, leading dimensions
// multiples of 8 elements, K > 0.
cudaError_t launch_gemm_bf16(const GemmArgs& args, cudaStream_t stream);

// Number of kernels this module has launched since load (for launch accounting).
uint64_t gemm_launch_count();

}  // namespace gemm
}  // namespace mgk
