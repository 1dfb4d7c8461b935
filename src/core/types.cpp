// Element sizes and printable names of the public enumerations.
// Sizes follow the reference table (src/core/common.cpp:19-38) with bf16 added.
#include "megray/types.h"

#include "megray/debug.h"

namespace MegRay {

size_t get_dtype_size(DType dtype) {
    static const size_t kSize[MEGRAY_DTYPE_COUNT] = {
            1 /*int8*/,  1 /*uint8*/, 4 /*int32*/, 4 /*uint32*/, 8 /*int64*/, 8 /*uint64*/,
            2 /*fp16*/,  4 /*fp32*/,  8 /*fp64*/,  1 /*char*/,   2 /*bf16*/};
    if (static_cast<int>(dtype) < 0 || dtype >= MEGRAY_DTYPE_COUNT)
        MEGRAY_THROW("unknown dtype");
    return kSize[dtype];
}

const char* status_name(Status s) {
    static const char* kName[MEGRAY_STATUS_COUNT] = {
            "OK",           "SYS_ERROR",        "CUDA_ERR",      "NCCL_ERR",       "UCX_ERR",
            "ENV_ERROR",    "INVALID_ARGUMENT", "INVALID_USAGE", "UNEXPECTED_ERR", "NOT_IMPLEMENTED",
            "HIP_ERR",      "RCCL_ERR",         "TIMEOUT",       "ABORTED",        "OUT_OF_BOUNDS"};
    if (static_cast<int>(s) < 0 || s >= MEGRAY_STATUS_COUNT)
        return "?";
    return kName[s];
}

const char* backend_name(Backend b) {
    static const char* kName[MEGRAY_BACKEND_COUNT] = {"NCCL", "UCX", "RCCL", "SHM", "NVL"};
    if (static_cast<int>(b) < 0 || b >= MEGRAY_BACKEND_COUNT)
        return "?";
    return kName[b];
}

const char* dtype_name(DType d) {
    static const char* kName[MEGRAY_DTYPE_COUNT] = {"int8",    "uint8",   "int32",   "uint32",
                                                    "int64",   "uint64",  "float16", "float32",
                                                    "float64", "char",    "bfloat16"};
    if (static_cast<int>(d) < 0 || d >= MEGRAY_DTYPE_COUNT)
        return "?";
    return kName[d];
}

const char* reduce_op_name(ReduceOp op) {
    static const char* kName[MEGRAY_REDUCEOP_COUNT] = {"sum", "max", "min"};
    if (static_cast<int>(op) < 0 || op >= MEGRAY_REDUCEOP_COUNT)
        return "?";
    return kName[op];
}

}  // namespace MegRay
