/**
 * Rendezvous client: one TCP connection to the server of a communicator group.
 *
 * Same calls and wire format as the reference client
 * (include/megray/client.h:24-49, src/core/client.cpp:28-139): connect sends
 * `u32 rank` and waits for the `u32` acknowledgement that the server sends once
 * all ranks are connected; barrier / broadcast / allgather are requests 1 / 2 /
 * 3.  Unlike the reference, connect gives up after a deadline instead of
 * retrying forever, every wait has a deadline, the socket is closed by the
 * destructor, and a lost server shows up as MEGRAY_SYS_ERROR / MEGRAY_TIMEOUT.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <mutex>

#include "megray/common.h"

namespace MegRay {

class Client {
public:
    Client(uint32_t nranks, uint32_t rank);
    ~Client();
    Client(const Client&) = delete;
    Client& operator=(const Client&) = delete;

    Status connect(const char* master_ip, int port);
    /** Close the connection; later calls return MEGRAY_INVALID_USAGE. */
    void close();
    bool connected() const { return m_connected; }

    /** Block until every rank has called barrier(). */
    Status barrier();

    /** `sendbuff` (read on root only) and `recvbuff` hold `sendlen` bytes. */
    Status broadcast(const void* sendbuff, void* recvbuff, size_t sendlen, uint32_t root);

    /** `sendbuff`: sendlen bytes; `recvbuff`: sendlen * nranks bytes, rank-major. */
    Status allgather(const void* sendbuff, void* recvbuff, size_t sendlen);

    /** Deadline of one wait in milliseconds (<= 0: wait forever). */
    void set_timeout_ms(int64_t ms) { m_timeout_ms = ms; }

    uint32_t nranks() const { return m_nranks; }
    uint32_t rank() const { return m_rank; }

private:
    uint32_t m_nranks;
    uint32_t m_rank;
    bool m_connected = false;
    int m_conn = -1;
    int64_t m_timeout_ms;
    int64_t m_connect_timeout_ms;
    std::mutex m_mutex;
};

}  // namespace MegRay
