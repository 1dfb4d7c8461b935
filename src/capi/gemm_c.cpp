// C entry points for the GEMM family (see include/megray/c_api.h).
#include "kernels/elementwise.cuh"
#include "kernels/gemm_tcgen05.cuh"
#include "kernels/launch_count.h"
#include <memory>

#include "megray/c_api.h"
#include "megray/communicator.h"
#include "nvl/fused_tp.h"

namespace {
mgk::gemm::GemmArgs to_gemm_args(const megray_gemm_args* a) {
    mgk::gemm::GemmArgs g{};
    g.A = a->A;
    g.B = a->B;
    g.D = a->D;
    g.D2 = a->D2;
    g.aux = a->aux;
    g.M = a->M;
    g.N = a->N;
    g.K = a->K;
    g.lda = a->lda;
    g.ldb = a->ldb;
    g.ldd = a->ldd;
    g.ldd2 = a->ldd2;
    g.ldaux = a->ldaux;
    g.a_mn = a->a_mn != 0;
    g.b_mn = a->b_mn != 0;
    g.epilogue = a->epilogue;
    g.aux_off = a->aux_off;
    g.m_rot = a->m_rot;
    g.sm_limit = a->sm_limit;
    g.variant = a->variant;
    g.a_ready = a->a_ready;
    g.rows_per_flag = a->rows_per_flag;
    g.a_ready_target = a->a_ready_target;
    g.peer_out = a->peer_out;
    g.rows_per_peer = a->rows_per_peer;
    g.grouped.m_block_group = a->m_block_group;
    g.grouped.group_rows_b = a->group_rows_b;
    g.grouped.k_begin = a->k_begin;
    g.grouped.k_end = a->k_end;
    g.grouped.groups = a->groups;
    g.error_flag = a->error_flag;
    g.wait_limit_ns = a->wait_limit_ns;
    return g;
}
struct CommBoxView {  // layout of the handle made by megray_comm_new (capi/comm_c.cpp)
    std::shared_ptr<MegRay::Communicator> comm;
};
}  // namespace

extern "C" int megray_gemm_tile_schedule(const megray_gemm_args* a, int sms, int* tiles, int max_tiles) {
    if (a == nullptr || tiles == nullptr)
        return -1;
    return mgk::gemm::tile_schedule(to_gemm_args(a), sms, tiles, max_tiles);
}

extern "C" int megray_gemm_bf16(const megray_gemm_args* a, void* stream) {
    if (a == nullptr)
        return 6;
    cudaError_t e = mgk::gemm::launch_gemm_bf16(to_gemm_args(a), static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

extern "C" int megray_tp_ag_gemm(void* comm, const megray_gemm_args* a, void* gather_buf, const void* shard_src,
                                 void* flags, void* stream) {
    if (comm == nullptr || a == nullptr)
        return 6;
    return MegRay::tp_ag_gemm(static_cast<CommBoxView*>(comm)->comm.get(), to_gemm_args(a), gather_buf, shard_src,
                              flags, static_cast<cudaStream_t>(stream));
}

extern "C" int megray_tp_gemm_rs(void* comm, const megray_gemm_args* a, void* staging, void* out,
                                 const void* residual, void* counters, size_t counter_bytes, void* stream) {
    if (comm == nullptr || a == nullptr)
        return 6;
    return MegRay::tp_gemm_rs(static_cast<CommBoxView*>(comm)->comm.get(), to_gemm_args(a), staging, out, residual,
                              counters, counter_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" size_t megray_tp_rs_counter_bytes(int shard_rows, int n_cols) {
    return MegRay::tp_rs_counter_bytes(shard_rows, n_cols);
}

extern "C" uint64_t megray_launch_count(void) { return mgk::launch_count(); }

extern "C" int megray_sgd_bf16(void* w, const void* g, float* momentum, uint64_t n, float lr, float mu,
                               float weight_decay, void* stream) {
    cudaError_t e = mgk::ew::launch_sgd_bf16(w, g, momentum, n, lr, mu, weight_decay,
                                             static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

extern "C" int megray_mse_bf16(const void* y, const void* target, void* dy, float* loss_out, uint64_t n,
                               float scale, void* stream) {
    cudaError_t e = mgk::ew::launch_mse_bf16(y, target, dy, loss_out, n, scale,
                                             static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

extern "C" int megray_add_rmsnorm_bf16(const void* x, const void* y, void* x_out, void* n_out, float* inv_rms,
                                       int rows, int cols, float eps, void* stream) {
    cudaError_t e = mgk::ew::launch_add_rmsnorm_bf16(x, y, x_out, n_out, inv_rms, rows, cols, eps,
                                                     static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

extern "C" int megray_rmsnorm_bwd_bf16(const void* dn, const void* n, const float* inv_rms, const void* dres,
                                       void* dx, int rows, int cols, void* stream) {
    cudaError_t e = mgk::ew::launch_rmsnorm_bwd_bf16(dn, n, inv_rms, dres, dx, rows, cols,
                                                     static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}
