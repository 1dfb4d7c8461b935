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

int megray_gemm_bf16(const megray_gemm_args* args, void* stream);

/* Kernels launched by this library since it was loaded (all modules). */
uint64_t megray_launch_count(void);

#ifdef __cplusplus
}
#endif
