// Rendezvous client.  Wire format (native byte order, no framing), identical to
// the reference client (src/core/client.cpp:56-60,75-80,95-111,125-136):
//   connect   : -> u32 rank                      <- u32 ack (after all ranks joined)
//   barrier   : -> u32 1                         <- u32 ack
//   broadcast : -> u32 2, u32 root, u64 len [+ len bytes from root]   <- len bytes
//   allgather : -> u32 3, u64 len, len bytes     <- len * nranks bytes
#include "megray/client.h"

#include <arpa/inet.h>
#include <errno.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include "megray/options.h"
#include "rendezvous/net.h"

namespace MegRay {

namespace {
enum : uint32_t { REQ_BARRIER = 1, REQ_BROADCAST = 2, REQ_ALLGATHER = 3 };
}

Client::Client(uint32_t nranks, uint32_t rank) : m_nranks(nranks), m_rank(rank) {
    const Options& o = global_options();
    m_timeout_ms = o.timeout_ms;
    m_connect_timeout_ms = o.connect_timeout_ms;
}

Client::~Client() { close(); }

void Client::close() {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (m_conn >= 0) {
        ::shutdown(m_conn, SHUT_RDWR);
        ::close(m_conn);
        m_conn = -1;
    }
    m_connected = false;
}

Status Client::connect(const char* master_ip, int port) {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (m_connected) {
        MEGRAY_ERROR("client already connected");
        return MEGRAY_INVALID_USAGE;
    }
    if (m_rank >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    struct sockaddr_in addr = {};
    addr.sin_family = AF_INET;
    addr.sin_port = htons(static_cast<uint16_t>(port));
    if (inet_pton(AF_INET, master_ip, &addr.sin_addr) != 1) {
        MEGRAY_ERROR("bad server address %s", master_ip);
        return MEGRAY_INVALID_ARGUMENT;
    }
    // The server may not be listening yet: retry until the deadline.
    const int64_t deadline = net::deadline_after(m_connect_timeout_ms);
    int fd = -1;
    for (;;) {
        fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (fd < 0) {
            MEGRAY_ERROR("socket: %s", strerror(errno));
            return MEGRAY_SYS_ERROR;
        }
        if (::connect(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) == 0)
            break;
        ::close(fd);
        fd = -1;
        if (deadline >= 0 && net::now_ms() >= deadline) {
            MEGRAY_ERROR("rank %u: no server at %s:%d after %lld ms", m_rank, master_ip, port,
                         static_cast<long long>(m_connect_timeout_ms));
            return MEGRAY_TIMEOUT;
        }
        usleep(50 * 1000);
    }
    net::tune_socket(fd);
    uint32_t rank = m_rank, ack = 1;
    Status s = net::send_all(fd, &rank, sizeof(rank), deadline);
    if (s == MEGRAY_OK)
        s = net::recv_all(fd, &ack, sizeof(ack), deadline);
    if (s == MEGRAY_OK && ack != 0) {
        MEGRAY_ERROR("server refused rank %u (code %u)", m_rank, ack);
        s = MEGRAY_SYS_ERROR;
    }
    if (s != MEGRAY_OK) {
        ::close(fd);
        return s;
    }
    m_conn = fd;
    m_connected = true;
    return MEGRAY_OK;
}

Status Client::barrier() {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (!m_connected)
        return MEGRAY_INVALID_USAGE;
    const int64_t dl = net::deadline_after(m_timeout_ms);
    uint32_t id = REQ_BARRIER, ack = 1;
    Status s = net::send_all(m_conn, &id, sizeof(id), dl);
    if (s == MEGRAY_OK)
        s = net::recv_all(m_conn, &ack, sizeof(ack), dl);
    if (s == MEGRAY_OK && ack != 0)
        s = MEGRAY_SYS_ERROR;
    return s;
}

Status Client::broadcast(const void* sendbuff, void* recvbuff, size_t len, uint32_t root) {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (!m_connected)
        return MEGRAY_INVALID_USAGE;
    if (root >= m_nranks || recvbuff == nullptr || (m_rank == root && sendbuff == nullptr && len))
        return MEGRAY_INVALID_ARGUMENT;
    const int64_t dl = net::deadline_after(m_timeout_ms);
    struct __attribute__((packed)) {
        uint32_t id, root;
        uint64_t len;
    } hdr = {REQ_BROADCAST, root, static_cast<uint64_t>(len)};
    Status s = net::send_all(m_conn, &hdr, sizeof(hdr), dl);
    if (s == MEGRAY_OK && m_rank == root)
        s = net::send_all(m_conn, sendbuff, len, dl);
    if (s == MEGRAY_OK)
        s = net::recv_all(m_conn, recvbuff, len, dl);
    return s;
}

Status Client::allgather(const void* sendbuff, void* recvbuff, size_t len) {
    std::lock_guard<std::mutex> lk(m_mutex);
    if (!m_connected)
        return MEGRAY_INVALID_USAGE;
    if ((sendbuff == nullptr || recvbuff == nullptr) && len)
        return MEGRAY_INVALID_ARGUMENT;
    const int64_t dl = net::deadline_after(m_timeout_ms);
    struct __attribute__((packed)) {
        uint32_t id;
        uint64_t len;
    } hdr = {REQ_ALLGATHER, static_cast<uint64_t>(len)};
    Status s = net::send_all(m_conn, &hdr, sizeof(hdr), dl);
    if (s == MEGRAY_OK)
        s = net::send_all(m_conn, sendbuff, len, dl);
    if (s == MEGRAY_OK)
        s = net::recv_all(m_conn, recvbuff, len * m_nranks, dl);
    return s;
}

}  // namespace MegRay
