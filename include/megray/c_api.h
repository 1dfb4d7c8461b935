/**
 * C interface of libmegray: what the Python package (ctypes) and other
 * non-C++ callers use.  Every function returns 0 on success; otherwise a
 * MegRay::Status value (positive) or, for the raw kernel launchers, the
 * negated cudaError_t.  Device pointers are passed as void*, streams as the
 * cudaStream_t handle value.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- tcgen05 bf16 GEMM family: D[M,N] = A[M,K] * B[N,K]^T ------------------ */
typedef struct {
    const void* A;
    const void* B;
    void* D;
    void* D2;        /* SwiGLU epilogue: H output */
    const void* aux; /* dSwiGLU epilogue: saved [G | U] */
    int M, N, K;
    int64_t lda, ldb, ldd, ldd2, ldaux;
    int a_mn, b_mn;  /* operand stored [K, rows] instead of [rows, K] */
    int epilogue;    /* 0 store, 1 swiglu, 2 dswiglu, 3 accumulate, 4 push to row owners */
    int aux_off;
    int m_rot;
    int sm_limit;
    int variant;     /* 0 automatic, 1 single-CTA 128x256 tile, 2 CTA-pair 256x256 tile, 3 CTA-pair 512x256 tile */
    const uint32_t* a_ready;
    int rows_per_flag;
    uint32_t a_ready_target;
    void* const* peer_out;
    int rows_per_peer;
    const int* m_block_group;
    int group_rows_b;
    const int* k_begin;
    const int* k_end;
    int groups;
    int* error_flag;
    uint64_t wait_limit_ns;
} megray_gemm_args;

/* Tile raster of a dense problem on a device with `sms` SMs, without a GPU: 4 ints per tile
 * (first row, first column, tile rows, output columns per tile) in launch order; returns the
 * number of tiles or -1. */
int megray_gemm_tile_schedule(const megray_gemm_args* a, int sms, int* tiles, int max_tiles);
int megray_gemm_bf16(const megray_gemm_args* args, void* stream);


/* ---- rendezvous ------------------------------------------------------------- */
int megray_get_host_ip(char* buf, size_t buflen);           /* 0 ok, 1 none */
int megray_get_free_port(void);                             /* port or -1 */
int megray_create_server(uint32_t nranks, int port);        /* free-function server */
void* megray_server_new(uint32_t nranks, int port);         /* RAII server; NULL on failure */
int megray_server_port(void* server);
int megray_server_running(void* server);
int megray_server_status(void* server);
uint64_t megray_server_requests(void* server);
void megray_server_stop(void* server);
void megray_server_delete(void* server);

void* megray_client_new(uint32_t nranks, uint32_t rank);
void megray_client_set_timeout_ms(void* client, int64_t ms);
int megray_client_connect(void* client, const char* ip, int port);
int megray_client_barrier(void* client);
int megray_client_broadcast(void* client, const void* send, void* recv, size_t len, uint32_t root);
int megray_client_allgather(void* client, const void* send, void* recv, size_t len);
void megray_client_delete(void* client);

/* ---- communicators ---------------------------------------------------------- */
/* ctx_type: 0 = host buffers (HostContext), 1 = CUDA stream (CudaContext, `stream` is the
 * cudaStream_t value).  dtype / op / backend take the MegRay enum values. */
void* megray_comm_new(uint32_t nranks, uint32_t rank, int backend); /* NULL: unknown backend */
void megray_comm_delete(void* comm);
int megray_comm_init(void* comm, const char* ip, int port);
int megray_comm_backend(void* comm);
int megray_comm_status(void* comm);
void megray_comm_abort(void* comm);
/* out[0..10) = calls, bytes, kernels, timeouts, oneshot, twoshot, nvls, copy, ll, direct */
void megray_comm_stats(void* comm, uint64_t* out);

int megray_send(void* comm, const void* buf, size_t len, int dtype, uint32_t peer, int ctx_type, void* stream);
int megray_recv(void* comm, void* buf, size_t len, int dtype, uint32_t peer, int ctx_type, void* stream);
int megray_scatter(void* comm, const void* send, void* recv, size_t recvlen, int dtype, uint32_t root, int ctx_type, void* stream);
int megray_gather(void* comm, const void* send, void* recv, size_t sendlen, int dtype, uint32_t root, int ctx_type, void* stream);
int megray_all_to_all(void* comm, const void* send, void* recv, size_t len, int dtype, int ctx_type, void* stream);
int megray_all_gather(void* comm, const void* send, void* recv, size_t sendlen, int dtype, int ctx_type, void* stream);
int megray_all_reduce(void* comm, const void* send, void* recv, size_t len, int dtype, int op, int ctx_type, void* stream);
int megray_reduce_scatter(void* comm, const void* send, void* recv, size_t recvlen, int dtype, int op, int ctx_type, void* stream);
int megray_broadcast(void* comm, const void* send, void* recv, size_t len, int dtype, uint32_t root, int ctx_type, void* stream);
int megray_reduce(void* comm, const void* send, void* recv, size_t len, int dtype, int op, uint32_t root, int ctx_type, void* stream);
int megray_group_start(void* comm);
int megray_group_end(void* comm);
int megray_host_barrier(void* comm);              /* host backend only */
void megray_host_set_timeout_ms(void* comm, int64_t ms);

/* ---- native NVLink backend extras (return 7 = INVALID_USAGE on other backends) ------- */
void* megray_nvl_alloc(void* comm, size_t bytes, size_t* offset_out);
int megray_nvl_free(void* comm, void* ptr);
void* megray_nvl_peer_ptr(void* comm, void* ptr, uint32_t peer);
/* Collective: make ordinary device memory reachable by the peers' kernels (single-pass paths). */
int megray_nvl_register(void* comm, void* ptr, size_t bytes);
int megray_nvl_deregister(void* comm, void* ptr);
void* megray_nvl_heap_base(void* comm, uint32_t peer);
size_t megray_nvl_heap_bytes(void* comm);
int megray_nvl_all_reduce_scaled(void* comm, const void* send, void* recv, size_t len, int in_dtype,
                                 int out_dtype, float scale, int op, void* stream);
int megray_nvl_stream_barrier(void* comm, void* stream);
void megray_nvl_set_device_timeout_ms(void* comm, int64_t ms);
/* verifies the guard zones around the staging workspaces; MEGRAY_OUT_OF_BOUNDS (14) if one was written */
int megray_nvl_check_canaries(void* comm);
/* send / recv: postpone the caller's stream's wait for the transfer until megray_nvl_p2p_join */
void megray_nvl_set_p2p_async(void* comm, int on);
int megray_nvl_p2p_join(void* comm, void* stream);

/* ---- host arithmetic (the oracle) and stand-alone device reduction ----------------------- */
int megray_cpu_reduce_n(const void* const* in, int n_in, void* out, size_t len, int dtype, int op);
/* Second oracle: replays the reference's ring all_reduce / binomial-tree reduce schedules over
 * host buffers (every pairwise step rounded to the element type). */
int megray_oracle_ring_all_reduce(const void* const* in, void* const* out, int nranks, size_t len, int dtype,
                                  int op);
int megray_oracle_tree_reduce(const void* const* in, void* out, int nranks, int root, size_t len, int dtype,
                              int op);
int megray_cpu_reduce_scale_cast(const void* const* in, int n_in, int in_dtype, void* out,
                                 int out_dtype, size_t len, int op, double scale);
int megray_reduce_n(const void* const* in, int n_in, void* out, size_t len, int in_dtype,
                    int out_dtype, int op, float scale, void* stream);

size_t megray_dtype_size(int dtype);   /* 0 for an unknown dtype */
void megray_set_log_level(int level);
void megray_trace_enable(const char* path);
size_t megray_trace_dump(void);

/* ---- tensor-parallel fused kernels (NVL communicators) ----------------------------------------
 * all_gather -> GEMM: A of `args` is ignored and replaced by `gather_buf` ([M, K], local, in the
 * symmetric heap); `shard_src` is this rank's [M/n, K] shard (in the heap, possibly its own rows of
 * gather_buf).  GEMM -> reduce_scatter: D of `args` is ignored; `staging` holds n slots of
 * [M/n, N]; `out` receives this rank's reduced [M/n, N] shard (+ residual).  `flags`: a 256-byte
 * zero-initialised block in the heap, the same block for every call on the same gather buffer.
 * `counters`: megray_tp_rs_counter_bytes(M/n, N) zero-initialised bytes in the heap (the same
 * offset on every rank), the same block for every call on the same staging buffer. */
int megray_tp_ag_gemm(void* comm, const megray_gemm_args* args, void* gather_buf, const void* shard_src,
                      void* flags, void* stream);
int megray_tp_gemm_rs(void* comm, const megray_gemm_args* args, void* staging, void* out,
                      const void* residual, void* counters, size_t counter_bytes, void* stream);
size_t megray_tp_rs_counter_bytes(int shard_rows, int n_cols);

/* ---- expert-parallel MoE kernels (src/kernels/moe.cuh) ---------------------------------------- */
int megray_moe_route(const float* logits, int tokens, int experts, int* idx, float* w, int* counts, void* stream);
int megray_moe_route_bwd(const int* idx, const float* w, const float* dw, int tokens, int experts,
                         float* dlogits, void* stream);
int megray_moe_plan(const int* counts_all, int nranks, int rank, int experts, int capacity_rows,
                    int* send_base, int* seg_begin, int* seg_end, int* seg_rows, int* block_group,
                    int* total, void* stream);
/* The plan with the exchange of the counts inside the launch (NVL communicators): `counts` are this
 * rank's per-expert counts; no separate all_gather is needed. */
int megray_moe_plan_exchange(void* comm, const int* counts, int experts, int capacity_rows, int* send_base,
                             int* seg_begin, int* seg_end, int* seg_rows, int* block_group, int* total, void* stream);
int megray_moe_zero_pads(void* buf, int row_elems, const int* seg_begin, const int* seg_rows,
                         const int* seg_end, int local_experts, void* stream);
/* peer_bufs: array of `nranks` device addresses (host array), one buffer per owner rank */
int megray_moe_dispatch(const void* src, int tokens, int row_elems, const int* idx, const float* w,
                        const int* send_base, int* cursor, const int* pos_in, int* pos_out,
                        void* const* peer_bufs, int nranks, int local_experts, int capacity_rows, void* stream);
int megray_moe_combine(void* out, int tokens, int row_elems, const int* idx, const float* w,
                       const int* pos, void* const* peer_bufs, int nranks, int local_experts, int capacity_rows, void* stream);
int megray_moe_combine_dw(const void* dout, int tokens, int row_elems, const int* idx, const int* pos,
                          void* const* peer_bufs, int nranks, int local_experts, int capacity_rows, float* dw, void* stream);

/* ---- training-harness kernels ---------------------------------------------------------------- */
int megray_sgd_bf16(void* w, const void* g, float* momentum, uint64_t n, float lr, float mu,
                    float weight_decay, void* stream);
int megray_mse_bf16(const void* y, const void* target, void* dy, float* loss_out, uint64_t n,
                    float scale, void* stream);

int megray_add_rmsnorm_bf16(const void* x, const void* y, void* x_out, void* n_out, float* inv_rms,
                            int rows, int cols, float eps, void* stream);
int megray_rmsnorm_bwd_bf16(const void* dn, const void* n, const float* inv_rms, const void* dres,
                            void* dx, int rows, int cols, void* stream);

/* Kernels launched by this library since it was loaded (all modules). */
uint64_t megray_launch_count(void);

#ifdef __cplusplus
}
#endif
