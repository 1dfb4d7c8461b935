/**
 * Rendezvous server.
 *
 * `get_host_ip`, `get_free_port` and `create_server` are the reference's free
 * functions (include/megray/server.h:19-24).  `Server` is the RAII form: the
 * service thread is joined by the destructor instead of being detached, and a
 * protocol violation or a lost rank ends the service (closing every
 * connection, which the clients report as MEGRAY_SYS_ERROR) rather than
 * terminating the process from a detached thread.
 */
#pragma once
#include <stdint.h>

#include <memory>

#include "megray/common.h"

namespace MegRay {

/** Address of the first non-loopback IPv4 interface (or of $MEGRAY_NET_DEVICE).
 *  The caller owns the returned array (delete[]), as in the reference. */
char* get_host_ip();

/** A TCP port that was free a moment ago. */
int get_free_port();

/** Start a server for `nranks` ranks on `port`; it lives until rank 0 disconnects. */
Status create_server(uint32_t nranks, int port);

class Server {
public:
    /** port == 0 picks a free port. Throws MegRay::Exception if the socket cannot be set up. */
    explicit Server(uint32_t nranks, int port = 0);
    ~Server();
    Server(const Server&) = delete;
    Server& operator=(const Server&) = delete;

    int port() const;
    uint32_t nranks() const;
    /** True while the service thread runs. */
    bool running() const;
    /** MEGRAY_OK, or why the service ended early. */
    Status status() const;
    /** Requests served so far (barriers + broadcasts + allgathers). */
    uint64_t requests_served() const;
    /** Ask the service to end now: closes all connections. */
    void stop();

    struct Impl;

private:
    std::shared_ptr<Impl> m_impl;
};

}  // namespace MegRay
