#include "nccl/nccl_communicator.h"

#include <cuda_runtime_api.h>

#include "megray/cuda_context.h"
#include "nccl/nccl_loader.h"

namespace MegRay {

struct NcclCommunicatorPrivate {
    ncclComm_t comm = nullptr;
    const nccl::Api* api = nullptr;
};

namespace {

#define NCCL_CHECK(expr)                                                               \
    do {                                                                               \
        ncclResult_t megray_nccl_ = (expr);                                            \
        if (megray_nccl_ != ncclSuccess) {                                             \
            MEGRAY_ERROR("nccl error [%d]: %s", megray_nccl_,                          \
                         m_nccl->api->GetErrorString(megray_nccl_));                   \
            return MEGRAY_NCCL_ERR;                                                    \
        }                                                                              \
    } while (0)

bool nccl_dtype(DType d, ncclDataType_t* out) {
    switch (d) {
        case MEGRAY_INT8: *out = ncclInt8; return true;
        case MEGRAY_UINT8: *out = ncclUint8; return true;
        case MEGRAY_INT32: *out = ncclInt32; return true;
        case MEGRAY_UINT32: *out = ncclUint32; return true;
        case MEGRAY_INT64: *out = ncclInt64; return true;
        case MEGRAY_UINT64: *out = ncclUint64; return true;
        case MEGRAY_FLOAT16: *out = ncclFloat16; return true;
        case MEGRAY_FLOAT32: *out = ncclFloat32; return true;
        case MEGRAY_FLOAT64: *out = ncclFloat64; return true;
        case MEGRAY_BFLOAT16: *out = ncclBfloat16; return true;
        case MEGRAY_CHAR: *out = ncclChar; return true;  // data movement only
        default: return false;
    }
}

bool nccl_op(ReduceOp op, ncclRedOp_t* out) {
    switch (op) {
        case MEGRAY_SUM: *out = ncclSum; return true;
        case MEGRAY_MAX: *out = ncclMax; return true;
        case MEGRAY_MIN: *out = ncclMin; return true;
        default: return false;
    }
}

}  // namespace

#define PREPARE(ctx)                                                                   \
    if (m_nccl->comm == nullptr) return MEGRAY_INVALID_USAGE;                          \
    if (m_aborted.load()) return MEGRAY_ABORTED;                                       \
    if (!(ctx) || (ctx)->type() != MEGRAY_CTX_CUDA) {                                  \
        MEGRAY_ERROR("NCCL backend needs a CudaContext");                              \
        return MEGRAY_INVALID_ARGUMENT;                                                \
    }                                                                                  \
    cudaStream_t stream = static_cast<CudaContext*>((ctx).get())->get_stream();        \
    m_stats.calls++

NcclCommunicator::NcclCommunicator(uint32_t nranks, uint32_t rank)
        : Communicator(nranks, rank), m_nccl(new NcclCommunicatorPrivate) {
    m_nccl->api = nccl::api();
}

NcclCommunicator::~NcclCommunicator() {
    if (m_nccl->comm != nullptr && m_nccl->api != nullptr) {
        if (m_aborted.load())
            m_nccl->api->CommAbort(m_nccl->comm);
        else
            m_nccl->api->CommDestroy(m_nccl->comm);
    }
}

size_t NcclCommunicator::unique_id_bytes() { return sizeof(ncclUniqueId); }

Status NcclCommunicator::finish_init(void* uid_ptr) {
    ncclUniqueId uid;
    memcpy(&uid, uid_ptr, sizeof(uid));
    NCCL_CHECK(m_nccl->api->CommInitRank(&m_nccl->comm, static_cast<int>(m_nranks), uid,
                                         static_cast<int>(m_rank)));
    return MEGRAY_OK;
}

Status NcclCommunicator::do_init() {
    if (m_nccl->api == nullptr)
        return MEGRAY_ENV_ERROR;
    ncclUniqueId uid;
    memset(&uid, 0, sizeof(uid));
    if (m_rank == 0)
        NCCL_CHECK(m_nccl->api->GetUniqueId(&uid));
    MEGRAY_CHECK(m_client->broadcast(&uid, &uid, sizeof(uid), 0));
    return finish_init(&uid);
}

Status NcclCommunicator::do_init(BcastCallback cb) {
    if (m_nccl->api == nullptr)
        return MEGRAY_ENV_ERROR;
    ncclUniqueId uid;
    memset(&uid, 0, sizeof(uid));
    if (m_rank == 0)
        NCCL_CHECK(m_nccl->api->GetUniqueId(&uid));
    cb(uid.internal, sizeof(uid));
    return finish_init(&uid);
}

Status NcclCommunicator::_send(const void* sendbuff, size_t size, uint32_t rank,
                               std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    m_stats.bytes += size;
    NCCL_CHECK(m_nccl->api->Send(sendbuff, size, ncclChar, static_cast<int>(rank), m_nccl->comm,
                                 stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::_recv(void* recvbuf, size_t size, uint32_t rank,
                               std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    m_stats.bytes += size;
    NCCL_CHECK(m_nccl->api->Recv(recvbuf, size, ncclChar, static_cast<int>(rank), m_nccl->comm,
                                 stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                                 uint32_t root, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t bytes = recvlen * get_dtype_size(dtype);
    m_stats.bytes += bytes;
    const nccl::Api* a = m_nccl->api;
    NCCL_CHECK(a->GroupStart());
    if (m_rank == root) {
        for (uint32_t r = 0; r < m_nranks; ++r)
            NCCL_CHECK(a->Send(static_cast<const char*>(sendbuff) + r * bytes, bytes, ncclChar,
                               static_cast<int>(r), m_nccl->comm, stream));
    }
    NCCL_CHECK(a->Recv(recvbuff, bytes, ncclChar, static_cast<int>(root), m_nccl->comm, stream));
    NCCL_CHECK(a->GroupEnd());
    return MEGRAY_OK;
}

Status NcclCommunicator::gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                                uint32_t root, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t bytes = sendlen * get_dtype_size(dtype);
    m_stats.bytes += bytes;
    const nccl::Api* a = m_nccl->api;
    NCCL_CHECK(a->GroupStart());
    if (m_rank == root) {
        for (uint32_t r = 0; r < m_nranks; ++r)
            NCCL_CHECK(a->Recv(static_cast<char*>(recvbuff) + r * bytes, bytes, ncclChar,
                               static_cast<int>(r), m_nccl->comm, stream));
    }
    NCCL_CHECK(a->Send(sendbuff, bytes, ncclChar, static_cast<int>(root), m_nccl->comm, stream));
    NCCL_CHECK(a->GroupEnd());
    return MEGRAY_OK;
}

Status NcclCommunicator::all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                    std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    const size_t bytes = len * get_dtype_size(dtype);
    m_stats.bytes += bytes;
    const nccl::Api* a = m_nccl->api;
    NCCL_CHECK(a->GroupStart());
    for (uint32_t r = 0; r < m_nranks; ++r) {
        NCCL_CHECK(a->Send(static_cast<const char*>(sendbuff) + r * bytes, bytes, ncclChar,
                           static_cast<int>(r), m_nccl->comm, stream));
        NCCL_CHECK(a->Recv(static_cast<char*>(recvbuff) + r * bytes, bytes, ncclChar,
                           static_cast<int>(r), m_nccl->comm, stream));
    }
    NCCL_CHECK(a->GroupEnd());
    return MEGRAY_OK;
}

Status NcclCommunicator::all_gather(const void* sendbuff, void* recvbuff, size_t sendlen,
                                    DType dtype, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    ncclDataType_t t;
    if (!nccl_dtype(dtype, &t))
        return MEGRAY_INVALID_ARGUMENT;
    m_stats.bytes += sendlen * get_dtype_size(dtype);
    NCCL_CHECK(m_nccl->api->AllGather(sendbuff, recvbuff, sendlen, t, m_nccl->comm, stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                    ReduceOp op, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    ncclDataType_t t;
    ncclRedOp_t o;
    if (dtype == MEGRAY_CHAR || !nccl_dtype(dtype, &t) || !nccl_op(op, &o))
        return MEGRAY_INVALID_ARGUMENT;
    m_stats.bytes += len * get_dtype_size(dtype);
    NCCL_CHECK(m_nccl->api->AllReduce(sendbuff, recvbuff, len, t, o, m_nccl->comm, stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen,
                                        DType dtype, ReduceOp op, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    ncclDataType_t t;
    ncclRedOp_t o;
    if (dtype == MEGRAY_CHAR || !nccl_dtype(dtype, &t) || !nccl_op(op, &o))
        return MEGRAY_INVALID_ARGUMENT;
    m_stats.bytes += recvlen * get_dtype_size(dtype);
    NCCL_CHECK(m_nccl->api->ReduceScatter(sendbuff, recvbuff, recvlen, t, o, m_nccl->comm, stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                   uint32_t root, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    ncclDataType_t t;
    if (root >= m_nranks || !nccl_dtype(dtype, &t))
        return MEGRAY_INVALID_ARGUMENT;
    m_stats.bytes += len * get_dtype_size(dtype);
    NCCL_CHECK(m_nccl->api->Broadcast(sendbuff, recvbuff, len, t, static_cast<int>(root),
                                      m_nccl->comm, stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                ReduceOp op, uint32_t root, std::shared_ptr<Context> ctx) {
    PREPARE(ctx);
    ncclDataType_t t;
    ncclRedOp_t o;
    if (root >= m_nranks || dtype == MEGRAY_CHAR || !nccl_dtype(dtype, &t) || !nccl_op(op, &o))
        return MEGRAY_INVALID_ARGUMENT;
    m_stats.bytes += len * get_dtype_size(dtype);
    NCCL_CHECK(m_nccl->api->Reduce(sendbuff, recvbuff, len, t, o, static_cast<int>(root),
                                   m_nccl->comm, stream));
    return MEGRAY_OK;
}

Status NcclCommunicator::group_start() {
    if (m_nccl->api == nullptr)
        return MEGRAY_ENV_ERROR;
    NCCL_CHECK(m_nccl->api->GroupStart());
    return MEGRAY_OK;
}

Status NcclCommunicator::group_end() {
    if (m_nccl->api == nullptr)
        return MEGRAY_ENV_ERROR;
    NCCL_CHECK(m_nccl->api->GroupEnd());
    return MEGRAY_OK;
}

void NcclCommunicator::abort() {
    Communicator::abort();
}

Status NcclCommunicator::status() {
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    if (m_nccl->comm != nullptr) {
        ncclResult_t async = ncclSuccess;
        if (m_nccl->api->CommGetAsyncError(m_nccl->comm, &async) != ncclSuccess ||
            (async != ncclSuccess && async != ncclInProgress))
            return MEGRAY_NCCL_ERR;
    }
    return MEGRAY_OK;
}

}  // namespace MegRay
