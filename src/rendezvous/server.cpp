// Rendezvous server: one service thread per communicator group.
//
// Protocol and request numbering are those of the reference server
// (src/core/server.cpp:99-265): ranks connect and send `u32 rank`; once all are
// in, each gets `u32 0`; then rounds of barrier(1) / broadcast(2) /
// allgather(3), every rank sending the same request, until rank 0 leaves.
//
// What differs from the reference: the thread is joinable and owned by a
// Server object (create_server keeps such objects in a process-wide list);
// every read has a deadline once a round has begun; a protocol violation, a
// lost rank or a deadline ends the service by closing all connections instead
// of throwing inside a detached thread; nranks == 1 works.
#include "megray/server.h"

#include <arpa/inet.h>
#include <errno.h>
#include <ifaddrs.h>
#include <net/if.h>
#include <netinet/in.h>
#include <poll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "megray/options.h"
#include "rendezvous/net.h"

namespace MegRay {

// ------------------------------------------------------------------ addresses

char* get_host_ip() {
    const std::string want = Options::from_env().net_device;
    if (want == "lo") {
        MEGRAY_ERROR("MEGRAY_NET_DEVICE must not be the loopback interface");
        return nullptr;
    }
    struct ifaddrs* list = nullptr;
    if (getifaddrs(&list) != 0) {
        MEGRAY_ERROR("getifaddrs: %s", strerror(errno));
        return nullptr;
    }
    char* out = nullptr;
    for (struct ifaddrs* it = list; it != nullptr && out == nullptr; it = it->ifa_next) {
        if (it->ifa_addr == nullptr || it->ifa_addr->sa_family != AF_INET)
            continue;
        if (it->ifa_flags & IFF_LOOPBACK)
            continue;
        if (!want.empty() && want != it->ifa_name)
            continue;
        char buf[INET_ADDRSTRLEN] = {0};
        auto* sin = reinterpret_cast<struct sockaddr_in*>(it->ifa_addr);
        if (inet_ntop(AF_INET, &sin->sin_addr, buf, sizeof(buf)) == nullptr)
            continue;
        out = new char[INET_ADDRSTRLEN];
        snprintf(out, INET_ADDRSTRLEN, "%s", buf);
    }
    freeifaddrs(list);
    if (out == nullptr)
        MEGRAY_ERROR("no usable IPv4 interface%s%s", want.empty() ? "" : " named ", want.c_str());
    return out;
}

int get_free_port() {
    int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0)
        return -1;
    struct sockaddr_in addr = {};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_ANY);
    addr.sin_port = 0;
    int port = -1;
    socklen_t len = sizeof(addr);
    if (::bind(fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) == 0 &&
        ::getsockname(fd, reinterpret_cast<struct sockaddr*>(&addr), &len) == 0)
        port = ntohs(addr.sin_port);
    ::close(fd);
    return port;
}

// ------------------------------------------------------------------ service

struct Server::Impl {
    uint32_t nranks = 0;
    int port = 0;
    int listen_fd = -1;
    int stop_fd = -1;  // eventfd: written by stop()
    std::thread thread;
    std::atomic<bool> running{false};
    std::atomic<int> status{MEGRAY_OK};
    std::atomic<uint64_t> served{0};
    std::vector<int> conns;
    int64_t timeout_ms = 0;

    ~Impl() {
        request_stop();
        if (thread.joinable())
            thread.join();
        if (listen_fd >= 0)
            ::close(listen_fd);
        if (stop_fd >= 0)
            ::close(stop_fd);
    }

    void request_stop() {
        if (stop_fd >= 0) {
            uint64_t one = 1;
            ssize_t r = ::write(stop_fd, &one, sizeof(one));
            (void)r;
        }
    }

    Status open(uint32_t n, int want_port) {
        nranks = n;
        timeout_ms = global_options().timeout_ms;
        listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
        if (listen_fd < 0)
            return MEGRAY_SYS_ERROR;
        int one = 1;
        setsockopt(listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
        struct sockaddr_in addr = {};
        addr.sin_family = AF_INET;
        addr.sin_addr.s_addr = htonl(INADDR_ANY);
        addr.sin_port = htons(static_cast<uint16_t>(want_port));
        if (::bind(listen_fd, reinterpret_cast<struct sockaddr*>(&addr), sizeof(addr)) != 0) {
            MEGRAY_ERROR("bind port %d: %s", want_port, strerror(errno));
            return MEGRAY_SYS_ERROR;
        }
        socklen_t len = sizeof(addr);
        getsockname(listen_fd, reinterpret_cast<struct sockaddr*>(&addr), &len);
        port = ntohs(addr.sin_port);
        if (::listen(listen_fd, static_cast<int>(n) + 8) != 0)
            return MEGRAY_SYS_ERROR;
        stop_fd = ::eventfd(0, EFD_CLOEXEC | EFD_NONBLOCK);
        if (stop_fd < 0)
            return MEGRAY_SYS_ERROR;
        running.store(true);
        thread = std::thread([this] { serve(); });
        return MEGRAY_OK;
    }

    void close_all() {
        for (int& fd : conns) {
            if (fd >= 0) {
                ::shutdown(fd, SHUT_RDWR);
                ::close(fd);
                fd = -1;
            }
        }
    }

    void fail(Status s, const char* why) {
        MEGRAY_ERROR("rendezvous server (port %d) ends: %s", port, why);
        status.store(s);
        close_all();
    }

    // Wait for activity: returns 1 when `fd` is readable, 0 on stop request, -1 on error.
    int wait_readable_or_stop(std::vector<struct pollfd>& pfds) {
        for (;;) {
            int r = ::poll(pfds.data(), pfds.size(), 1000);
            if (r < 0 && errno != EINTR)
                return -1;
            if (r <= 0)
                continue;
            if (pfds[0].revents)  // stop_fd is always entry 0
                return 0;
            return 1;
        }
    }

    bool accept_all() {
        conns.assign(nranks, -1);
        uint32_t joined = 0;
        while (joined < nranks) {
            std::vector<struct pollfd> pfds = {{stop_fd, POLLIN, 0}, {listen_fd, POLLIN, 0}};
            int w = wait_readable_or_stop(pfds);
            if (w <= 0) {
                if (w < 0)
                    fail(MEGRAY_SYS_ERROR, "poll failed while accepting");
                else
                    close_all();
                return false;
            }
            int fd = ::accept(listen_fd, nullptr, nullptr);
            if (fd < 0)
                continue;
            net::tune_socket(fd);
            uint32_t rank = 0;
            // a connection that never names its rank must not block the others for long
            Status s = net::recv_all(fd, &rank, sizeof(rank), net::deadline_after(5000));
            if (s != MEGRAY_OK || rank >= nranks || conns[rank] >= 0) {
                MEGRAY_WARN("rendezvous server: dropped a connection (bad or duplicate rank %u)",
                            rank);
                uint32_t nack = 1;
                net::send_all(fd, &nack, sizeof(nack), net::deadline_after(1000));
                ::close(fd);
                continue;
            }
            conns[rank] = fd;
            ++joined;
        }
        uint32_t ack = 0;
        for (uint32_t r = 0; r < nranks; ++r) {
            if (net::send_all(conns[r], &ack, sizeof(ack), net::deadline_after(timeout_ms)) !=
                MEGRAY_OK) {
                fail(MEGRAY_SYS_ERROR, "a rank left before the group was complete");
                return false;
            }
        }
        return true;
    }

    void serve() {
        if (accept_all())
            rounds();
        close_all();
        running.store(false);
    }

    void rounds() {
        std::vector<uint32_t> ids(nranks);
        for (;;) {
            // idle: wait without deadline for the first request (or a departure)
            std::vector<struct pollfd> pfds;
            pfds.push_back({stop_fd, POLLIN, 0});
            for (uint32_t r = 0; r < nranks; ++r)
                if (conns[r] >= 0)
                    pfds.push_back({conns[r], POLLIN, 0});
            if (pfds.size() == 1)
                return;  // everybody left
            int w = wait_readable_or_stop(pfds);
            if (w == 0)
                return;
            if (w < 0) {
                fail(MEGRAY_SYS_ERROR, "poll failed");
                return;
            }
            // Sort out what woke us: departures (EOF) versus a request.
            bool request = false;
            for (size_t i = 1; i < pfds.size(); ++i) {
                if (!pfds[i].revents)
                    continue;
                uint32_t r = 0;
                while (conns[r] != pfds[i].fd)
                    ++r;
                if (alive(r))
                    request = true;
            }
            if (conns[0] < 0)
                return;  // rank 0 closing between rounds is the regular end of service
            if (!request)
                continue;  // some other rank left; idle ranks are still served
            // A round has begun: every rank must show up before the deadline.
            const int64_t dl = net::deadline_after(timeout_ms);
            for (uint32_t r = 0; r < nranks; ++r) {
                if (conns[r] < 0) {
                    fail(MEGRAY_SYS_ERROR, "request after a rank has left the group");
                    return;
                }
                Status s = net::recv_all(conns[r], &ids[r], sizeof(uint32_t), dl, nullptr, stop_fd);
                if (s != MEGRAY_OK) {
                    fail(s, s == MEGRAY_TIMEOUT ? "a rank did not join the round in time"
                                                : "lost a rank in the middle of a round");
                    return;
                }
            }
            for (uint32_t r = 1; r < nranks; ++r) {
                if (ids[r] != ids[0]) {
                    fail(MEGRAY_INVALID_ARGUMENT, "ranks disagree on the request");
                    return;
                }
            }
            Status s;
            switch (ids[0]) {
                case 1:
                    s = serve_barrier(dl);
                    break;
                case 2:
                    s = serve_broadcast(dl);
                    break;
                case 3:
                    s = serve_allgather(dl);
                    break;
                default:
                    s = MEGRAY_INVALID_ARGUMENT;
            }
            if (s != MEGRAY_OK) {
                fail(s, "request failed (size/root mismatch, lost rank or deadline)");
                return;
            }
            served.fetch_add(1);
        }
    }

    // Peek at rank r's socket: false (and the slot is cleared) if the peer has closed.
    bool alive(uint32_t r) {
        if (conns[r] < 0)
            return false;
        char c;
        ssize_t n = ::recv(conns[r], &c, 1, MSG_PEEK | MSG_DONTWAIT);
        if (n == 0) {
            ::close(conns[r]);
            conns[r] = -1;
            return false;
        }
        return true;
    }

    Status serve_barrier(int64_t dl) {
        uint32_t ack = 0;
        for (uint32_t r = 0; r < nranks; ++r)
            MEGRAY_CHECK(net::send_all(conns[r], &ack, sizeof(ack), dl, stop_fd));
        return MEGRAY_OK;
    }

    Status serve_broadcast(int64_t dl) {
        uint32_t root0 = 0;
        uint64_t len0 = 0;
        for (uint32_t r = 0; r < nranks; ++r) {
            struct __attribute__((packed)) {
                uint32_t root;
                uint64_t len;
            } h;
            MEGRAY_CHECK(net::recv_all(conns[r], &h, sizeof(h), dl, nullptr, stop_fd));
            if (r == 0) {
                root0 = h.root;
                len0 = h.len;
            } else if (h.root != root0 || h.len != len0) {
                MEGRAY_ERROR("broadcast: rank %u sent root %u len %llu, rank 0 sent root %u len %llu",
                             r, h.root, static_cast<unsigned long long>(h.len), root0,
                             static_cast<unsigned long long>(len0));
                return MEGRAY_INVALID_ARGUMENT;
            }
        }
        if (root0 >= nranks || len0 > (1ull << 32))
            return MEGRAY_INVALID_ARGUMENT;
        std::vector<char> data(len0);
        MEGRAY_CHECK(net::recv_all(conns[root0], data.data(), len0, dl, nullptr, stop_fd));
        for (uint32_t r = 0; r < nranks; ++r)
            MEGRAY_CHECK(net::send_all(conns[r], data.data(), len0, dl, stop_fd));
        return MEGRAY_OK;
    }

    Status serve_allgather(int64_t dl) {
        uint64_t len0 = 0;
        std::vector<char> data;
        for (uint32_t r = 0; r < nranks; ++r) {
            uint64_t len = 0;
            MEGRAY_CHECK(net::recv_all(conns[r], &len, sizeof(len), dl, nullptr, stop_fd));
            if (r == 0) {
                len0 = len;
                if (len0 > (1ull << 32) / nranks)
                    return MEGRAY_INVALID_ARGUMENT;
                data.resize(len0 * nranks);
            } else if (len != len0) {
                MEGRAY_ERROR("allgather: rank %u sent len %llu, rank 0 sent %llu", r,
                             static_cast<unsigned long long>(len),
                             static_cast<unsigned long long>(len0));
                return MEGRAY_INVALID_ARGUMENT;
            }
            MEGRAY_CHECK(net::recv_all(conns[r], data.data() + r * len0, len0, dl, nullptr, stop_fd));
        }
        for (uint32_t r = 0; r < nranks; ++r)
            MEGRAY_CHECK(net::send_all(conns[r], data.data(), data.size(), dl, stop_fd));
        return MEGRAY_OK;
    }
};

Server::Server(uint32_t nranks, int port) : m_impl(std::make_shared<Impl>()) {
    if (nranks == 0)
        MEGRAY_THROW("Server: nranks must be positive");
    if (m_impl->open(nranks, port) != MEGRAY_OK)
        MEGRAY_THROW("Server: cannot listen");
}

Server::~Server() = default;

int Server::port() const { return m_impl->port; }
uint32_t Server::nranks() const { return m_impl->nranks; }
bool Server::running() const { return m_impl->running.load(); }
Status Server::status() const { return static_cast<Status>(m_impl->status.load()); }
uint64_t Server::requests_served() const { return m_impl->served.load(); }
void Server::stop() { m_impl->request_stop(); }

// Servers started through the free function live here until they finish (or
// the process exits): finished ones are joined on the next call.
namespace {
std::mutex g_servers_mu;
std::vector<std::shared_ptr<Server::Impl>>& g_servers() {
    static std::vector<std::shared_ptr<Server::Impl>> v;
    return v;
}
}  // namespace

Status create_server(uint32_t nranks, int port) {
    if (nranks == 0 || port <= 0)
        return MEGRAY_INVALID_ARGUMENT;
    auto impl = std::make_shared<Server::Impl>();
    MEGRAY_CHECK(impl->open(nranks, port));
    std::lock_guard<std::mutex> lk(g_servers_mu);
    auto& v = g_servers();
    for (size_t i = 0; i < v.size();) {
        if (!v[i]->running.load())
            v.erase(v.begin() + static_cast<long>(i));  // joins in ~Impl
        else
            ++i;
    }
    v.push_back(impl);
    return MEGRAY_OK;
}

}  // namespace MegRay
