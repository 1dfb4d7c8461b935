// Tensor-parallel fused entry points of the NVL backend: all_gather -> GEMM and
// GEMM -> reduce_scatter as single kernels (kernels/gemm_tcgen05.cu) that move the
// activation shards over NVLink while the tensor cores run.
//
//   ag_gemm : D = epilogue( gather(A shards)[T, K] * B^T ).  The kernel's communication warps
//             pull every peer's [T/n, K] shard from that peer's memory into the local gather
//             buffer (own shard first, then rank+1, ...) and publish one ready word per shard;
//             the TMA producer waits for the word of the shard that owns its rows, so tiles
//             of a shard start as soon as that shard has landed.
//   gemm_rs : out[T/n, N] = sum over ranks of (A * B^T)[rows of this rank].  The epilogue
//             stores each partial tile of another rank's rows straight into that rank's
//             staging slot over NVLink and counts it there; the tiles of the rank's own rows
//             come last, and their epilogue adds the staged partials of the other ranks (in
//             rank order) to its accumulator and writes the shard.  No separate reduction pass.
//
// The reference offers only the separate all_gather / reduce_scatter calls
// (include/megray/communicator.h:79-95) around whatever GEMM its user runs.
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#include "kernels/gemm_tcgen05.cuh"
#include "megray/communicator.h"

namespace MegRay {

/** Bytes of the flag block a gather buffer needs (symmetric-heap memory, zeroed once). */
constexpr size_t kTpFlagBytes = 256;
/** Bytes of the delivery counters a reduce_scatter staging buffer needs (symmetric-heap memory at
 *  the same offset on every rank, zeroed once): one word per 32 rows x 256 columns of a shard. */
size_t tp_rs_counter_bytes(int shard_rows, int n_cols);

/**
 * all_gather -> GEMM.  `g` describes the GEMM with A = `gather_buf` (this rank's local [T, K]
 * buffer in the symmetric heap, M = T); `shard_src` is this rank's [T/n, K] shard (in the heap;
 * it may be the rank's own rows of `gather_buf`); `flags` a kTpFlagBytes block in the heap at the
 * same offset on every rank.  Collective: all ranks call it in the same order.
 */
Status tp_ag_gemm(Communicator* comm, mgk::gemm::GemmArgs g, void* gather_buf, const void* shard_src,
                  void* flags, cudaStream_t stream);

/**
 * GEMM -> reduce_scatter.  `g` describes the GEMM whose [T, N] result is reduced over ranks
 * (its D is ignored); `staging` is n slots of [T/n, N] bf16 in the heap (same offset on every
 * rank); `counters` is tp_rs_counter_bytes(T/n, N) bytes in the heap, used by every call on this
 * staging buffer; `out` receives this rank's [T/n, N] shard (+ `residual` if non-null).
 */
Status tp_gemm_rs(Communicator* comm, mgk::gemm::GemmArgs g, void* staging, void* out,
                  const void* residual, void* counters, size_t counter_bytes, cudaStream_t stream);

}  // namespace MegRay
