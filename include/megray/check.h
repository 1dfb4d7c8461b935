/**
 * Error-propagation macros: each comes as a pair, one that returns a Status
 * from the enclosing function (..._CHECK) and one that throws (..._ASSERT).
 * Names match the reference (include/megray/common.h:39-96,
 * include/megray/cuda_context.h:24-42) so that backend code written against it
 * compiles unchanged.
 */
#pragma once
#include <errno.h>
#include <string.h>

#include "megray/debug.h"
#include "megray/types.h"

#define MEGRAY_CHECK(expr)                                                             \
    do {                                                                               \
        MegRay::Status megray_status_ = (expr);                                        \
        if (megray_status_ != MegRay::MEGRAY_OK) {                                     \
            MEGRAY_ERROR("error [%d] %s", megray_status_,                              \
                         MegRay::status_name(megray_status_));                         \
            return megray_status_;                                                     \
        }                                                                              \
    } while (0)

#define SYS_CHECK_RET(expr, errval, retval)                                    \
    do {                                                                       \
        retval = (expr);                                                       \
        if (retval == errval) {                                                \
            MEGRAY_ERROR("system error [%d]: %s", errno, strerror(errno));     \
            return MegRay::MEGRAY_SYS_ERROR;                                   \
        }                                                                      \
    } while (0)

#define SYS_CHECK(expr, errval)                      \
    do {                                             \
        int megray_ret_;                             \
        SYS_CHECK_RET(expr, errval, megray_ret_);    \
    } while (0)

#define SYS_ASSERT_RET(expr, errval, retval)                                   \
    do {                                                                       \
        retval = (expr);                                                       \
        if (retval == errval) {                                                \
            MEGRAY_ERROR("system error [%d]: %s", errno, strerror(errno));     \
            MEGRAY_THROW("system error");                                      \
        }                                                                      \
    } while (0)

#define SYS_ASSERT(expr, errval)                     \
    do {                                             \
        int megray_ret_;                             \
        SYS_ASSERT_RET(expr, errval, megray_ret_);   \
    } while (0)

#ifdef MEGRAY_WITH_CUDA
#include <cuda_runtime_api.h>

#ifndef CUDA_CHECK
#define CUDA_CHECK(expr)                                                       \
    do {                                                                       \
        cudaError_t megray_cuda_ = (expr);                                     \
        if (megray_cuda_ != cudaSuccess) {                                     \
            MEGRAY_ERROR("cuda error [%d]: %s", megray_cuda_,                  \
                         cudaGetErrorString(megray_cuda_));                    \
            return MegRay::MEGRAY_CUDA_ERR;                                    \
        }                                                                      \
    } while (0)
#endif

#ifndef CUDA_ASSERT
#define CUDA_ASSERT(expr)                                                      \
    do {                                                                       \
        cudaError_t megray_cuda_ = (expr);                                     \
        if (megray_cuda_ != cudaSuccess) {                                     \
            MEGRAY_ERROR("cuda error [%d]: %s", megray_cuda_,                  \
                         cudaGetErrorString(megray_cuda_));                    \
            MEGRAY_THROW("cuda error");                                        \
        }                                                                      \
    } while (0)
#endif
#endif  // MEGRAY_WITH_CUDA
