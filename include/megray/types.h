/**
 * Enumerations of the public interface.  Numeric values 0..9 / 0..3 / 0..2 are
 * those of the reference (include/megray/common.h:23-37,98-127) so that code
 * and serialized values written against it keep working; new members are
 * appended.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace MegRay {

typedef enum {
    MEGRAY_OK = 0,
    MEGRAY_SYS_ERROR = 1,
    MEGRAY_CUDA_ERR = 2,
    MEGRAY_NCCL_ERR = 3,
    MEGRAY_UCX_ERR = 4,
    MEGRAY_ENV_ERROR = 5,
    MEGRAY_INVALID_ARGUMENT = 6,
    MEGRAY_INVALID_USAGE = 7,
    MEGRAY_UNEXPECTED_ERR = 8,
    MEGRAY_NOT_IMPLEMENTED = 9,
    MEGRAY_HIP_ERR = 10,
    MEGRAY_RCCL_ERR = 11,
    MEGRAY_TIMEOUT = 12,  /* a bounded wait (host or device) ran out */
    MEGRAY_ABORTED = 13,  /* the communicator was aborted */
    MEGRAY_OUT_OF_BOUNDS = 14, /* a bounds-checked build caught an access outside the call's buffers */
    MEGRAY_STATUS_COUNT = 15,
} Status;

typedef enum {
    MEGRAY_NCCL = 0,
    MEGRAY_UCX = 1,
    MEGRAY_RCCL = 2,
    MEGRAY_SHM = 3,
    MEGRAY_NVL = 4, /* native NVLink 5 / NVSwitch backend */
    MEGRAY_BACKEND_COUNT = 5,
} Backend;

typedef enum {
    MEGRAY_INT8 = 0,
    MEGRAY_UINT8 = 1,
    MEGRAY_INT32 = 2,
    MEGRAY_UINT32 = 3,
    MEGRAY_INT64 = 4,
    MEGRAY_UINT64 = 5,
    MEGRAY_FLOAT16 = 6,
    MEGRAY_FLOAT32 = 7,
    MEGRAY_FLOAT64 = 8,
    MEGRAY_CHAR = 9, /* bytes: data movement only, no reductions */
    MEGRAY_BFLOAT16 = 10,
    MEGRAY_DTYPE_COUNT = 11,
} DType;

typedef enum {
    MEGRAY_SUM = 0,
    MEGRAY_MAX = 1,
    MEGRAY_MIN = 2,
    MEGRAY_REDUCEOP_COUNT = 3,
} ReduceOp;

/** Bytes per element; throws MegRay::Exception for an unknown dtype. */
size_t get_dtype_size(DType dtype);

/** Printable names (never null). */
const char* status_name(Status s);
const char* backend_name(Backend b);
const char* dtype_name(DType d);
const char* reduce_op_name(ReduceOp op);

}  // namespace MegRay
