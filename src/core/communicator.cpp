// Backend-independent part of Communicator: initialisation through the
// rendezvous server or a caller-supplied broadcast, and the element-count to
// byte-count step of send/recv (reference src/core/communicator.cpp:17-37).
#include "megray/communicator.h"

#include "megray/options.h"

namespace MegRay {

Status Communicator::init(const char* master_ip, int port) {
    if (master_ip == nullptr)
        return MEGRAY_INVALID_ARGUMENT;
    set_log_rank(static_cast<int>(m_rank));
    m_client = std::make_shared<Client>(m_nranks, m_rank);
    MEGRAY_CHECK(m_client->connect(master_ip, port));
    return do_init();
}

Status Communicator::init(BcastCallback cb) {
    if (!cb)
        return MEGRAY_INVALID_ARGUMENT;
    set_log_rank(static_cast<int>(m_rank));
    return do_init(cb);
}

Status Communicator::send(const void* sendbuff, size_t len, DType dtype, uint32_t rank,
                          std::shared_ptr<Context> ctx) {
    if (rank >= m_nranks || rank == m_rank)
        return MEGRAY_INVALID_ARGUMENT;
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    return _send(sendbuff, len * get_dtype_size(dtype), rank, ctx);
}

Status Communicator::recv(void* recvbuf, size_t len, DType dtype, uint32_t rank,
                          std::shared_ptr<Context> ctx) {
    if (rank >= m_nranks || rank == m_rank)
        return MEGRAY_INVALID_ARGUMENT;
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    return _recv(recvbuf, len * get_dtype_size(dtype), rank, ctx);
}

}  // namespace MegRay
