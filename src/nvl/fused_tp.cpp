#include "nvl/fused_tp.h"

#include "megray/fused.h"
#include "megray/trace.h"

namespace MegRay {

namespace {
struct FlagBlock {
    uint32_t ag_ready[8];
    uint32_t ag_count[8];
    uint32_t ag_start[8];
};
}  // namespace

size_t tp_rs_counter_bytes(int shard_rows, int n_cols) {
    return static_cast<size_t>((shard_rows + 31) / 32) * static_cast<size_t>((n_cols + 255) / 256) * sizeof(uint32_t);
}

Status tp_ag_gemm(Communicator* comm, mgk::gemm::GemmArgs g, void* gather_buf, const void* shard_src,
                  void* flags, cudaStream_t stream) {
    NvlInterface* nvl = as_nvl(comm);
    if (nvl == nullptr)
        return MEGRAY_INVALID_USAGE;
    const int n = static_cast<int>(comm->nranks()), rank = static_cast<int>(comm->rank());
    if (g.a_mn || g.M % n || !nvl->in_heap(gather_buf, 1) || !nvl->in_heap(shard_src, 1) ||
        !nvl->in_heap(flags, kTpFlagBytes))
        return MEGRAY_INVALID_ARGUMENT;
    MEGRAY_CHECK(nvl->fused_begin(stream));
    TraceScope trace("tp_ag_gemm", static_cast<size_t>(g.M) * g.K * 2, comm->rank());
    const int shard_rows = g.M / n;
    const size_t row_bytes = static_cast<size_t>(g.lda) * 2;
    if (g.lda != g.K || shard_rows % 128)
        return MEGRAY_INVALID_ARGUMENT;  // rows must be contiguous; shards are whole row blocks
    const size_t shard_bytes = static_cast<size_t>(shard_rows) * row_bytes;
    char* gb = static_cast<char*>(gather_buf);
    const bool in_place = shard_src == gb + static_cast<size_t>(rank) * shard_bytes;
    auto* fb = static_cast<FlagBlock*>(flags);

    mgk::gemm::FuseArgs& f = g.fuse;
    f.nranks = n;
    f.rank = rank;
    f.shard_rows = shard_rows;
    f.row_bytes = static_cast<int>(row_bytes);
    f.epoch = nvl->reserve_epochs(1) + 1;
    f.ag_dst = gather_buf;
    for (int q = 0; q < n; ++q) {
        if (in_place)
            f.ag_src[q] = static_cast<char*>(nvl->peer_ptr(gb, q)) + static_cast<size_t>(q) * shard_bytes;
        else
            f.ag_src[q] = nvl->peer_ptr(const_cast<void*>(shard_src), q);
        f.ag_start_peer[q] = static_cast<FlagBlock*>(nvl->peer_ptr(fb, q))->ag_start;
    }
    if (in_place)
        f.ag_src[rank] = nullptr;  // already where it belongs
    else
        f.ag_src[rank] = shard_src;
    f.ag_ready = fb->ag_ready;
    f.ag_count = fb->ag_count;
    f.ag_start_local = fb->ag_start;
    g.A = gather_buf;
    g.a_ready = fb->ag_ready;
    g.rows_per_flag = shard_rows;
    g.a_ready_target = f.epoch;
    g.m_rot = rank * shard_rows;  // own shard first, then in the order the shards arrive
    if (g.wait_limit_ns == 0)
        g.wait_limit_ns = nvl->device_timeout_ns();
    g.comm_status = nvl->status_word();
    cudaError_t e = mgk::gemm::launch_gemm_bf16(g, stream);
    if (e != cudaSuccess) {
        MEGRAY_ERROR("tp_ag_gemm launch: %s", cudaGetErrorString(e));
        return MEGRAY_CUDA_ERR;
    }
    nvl->fused_end(stream);
    return MEGRAY_OK;
}

Status tp_gemm_rs(Communicator* comm, mgk::gemm::GemmArgs g, void* staging, void* out,
                  const void* residual, void* counters, size_t counter_bytes, cudaStream_t stream) {
    NvlInterface* nvl = as_nvl(comm);
    if (nvl == nullptr)
        return MEGRAY_INVALID_USAGE;
    const int n = static_cast<int>(comm->nranks()), rank = static_cast<int>(comm->rank());
    if (g.M % n || out == nullptr)
        return MEGRAY_INVALID_ARGUMENT;
    const int shard_rows = g.M / n;
    if (shard_rows % 256 || g.N % 8)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t row_bytes = static_cast<size_t>(g.N) * 2;
    const size_t shard_bytes = static_cast<size_t>(shard_rows) * row_bytes;
    const size_t need = tp_rs_counter_bytes(shard_rows, g.N);
    if (counter_bytes < need || !nvl->in_heap(counters, need) || !nvl->in_heap(staging, shard_bytes * n)) {
        MEGRAY_ERROR("tp_gemm_rs: staging (%zu bytes) and counters (%zu bytes) must lie in the symmetric heap",
                     shard_bytes * n, need);
        return MEGRAY_INVALID_ARGUMENT;
    }
    MEGRAY_CHECK(nvl->fused_begin(stream));
    TraceScope trace("tp_gemm_rs", static_cast<size_t>(g.M) * g.N * 2, comm->rank());
    auto* cnt = static_cast<uint32_t*>(counters);

    // every piece of 32 rows x 256 columns of this rank's shard is delivered once by each other
    // rank in each call; the counters are cumulative over the calls on this block
    const uint32_t calls = nvl->fused_call_count(counters);
    mgk::gemm::FuseArgs& f = g.fuse;
    f.nranks = n;
    f.rank = rank;
    f.shard_rows = shard_rows;
    f.row_bytes = static_cast<int>(row_bytes);
    f.epoch = 0;
    for (int p = 0; p < n; ++p) {
        f.rs_peer_out[p] = static_cast<char*>(nvl->peer_ptr(staging, p)) + static_cast<size_t>(rank) * shard_bytes;
        f.rs_count_peer[p] = static_cast<uint32_t*>(nvl->peer_ptr(cnt, p));
    }
    f.rs_count_local = cnt;
    f.rs_col_tiles = (g.N + 255) / 256;
    f.rs_target = static_cast<uint32_t>(n - 1) * calls;
    f.rs_stage_local = staging;
    f.rs_out = out;
    f.rs_residual = residual;
    g.epilogue = mgk::gemm::EPI_PUSH;
    g.D = staging;  // unused by the push epilogue, but must be a valid aligned address
    g.ldd = g.N;
    g.peer_out = nullptr;
    g.rows_per_peer = shard_rows;
    g.m_rot = ((rank + 1) % n) * shard_rows;  // rows of remote owners first, own rows last
    if (g.wait_limit_ns == 0)
        g.wait_limit_ns = nvl->device_timeout_ns();
    g.comm_status = nvl->status_word();
    cudaError_t e = mgk::gemm::launch_gemm_bf16(g, stream);
    if (e != cudaSuccess) {
        MEGRAY_ERROR("tp_gemm_rs launch: %s", cudaGetErrorString(e));
        return MEGRAY_CUDA_ERR;
    }
    nvl->fused_end(stream);
    return MEGRAY_OK;
}

}  // namespace MegRay
