/**
 * The communicator interface.
 *
 * Signatures, buffer-length contracts and the split into public element-count
 * calls and protected byte-count `_send/_recv` are the reference's
 * (include/megray/communicator.h:32-123).  Added on top: abort()/status(),
 * per-communicator statistics, and a backend() query.
 *
 * Length contracts (elements of `dtype`), n = nranks:
 *   scatter         send n*recvlen (root only, may be null elsewhere) -> recv recvlen
 *   gather          send sendlen -> recv n*sendlen (root only, may be null elsewhere)
 *   all_to_all      send n*len -> recv n*len; chunk r goes to / comes from rank r
 *   all_gather      send sendlen -> recv n*sendlen
 *   all_reduce      send len -> recv len
 *   reduce_scatter  send n*recvlen -> recv recvlen
 *   broadcast       send len (root) -> recv len (every rank, root included)
 *   reduce          send len -> recv len (root only)
 * CUDA backends enqueue on the context's stream and return; the caller
 * synchronises the stream.
 */
#pragma once
#include <atomic>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "megray/client.h"
#include "megray/common.h"
#include "megray/context.h"

namespace MegRay {

/** Caller-supplied broadcast of a small blob from rank 0, in place. */
using BcastCallback = std::function<void(char*, size_t len)>;

/** Counters a communicator keeps about its own activity. */
struct CommStats {
    uint64_t calls = 0;         /* collective / p2p calls issued */
    uint64_t bytes = 0;         /* payload bytes of those calls (per-rank unit) */
    uint64_t kernels = 0;       /* kernels of this library launched */
    uint64_t timeouts = 0;      /* bounded waits that ran out */
    uint64_t algo_oneshot = 0;  /* calls served by each algorithm family */
    uint64_t algo_twoshot = 0;
    uint64_t algo_nvls = 0;
    uint64_t algo_copy = 0;
    uint64_t algo_ll = 0;       /* small messages as flagged words (no barrier) */
    uint64_t algo_direct = 0;   /* single-pass kernels on the peers' buffers themselves */
};

class Communicator {
public:
    Communicator(uint32_t nranks, uint32_t rank) : m_nranks(nranks), m_rank(rank) {}
    virtual ~Communicator() = default;

    uint32_t nranks() { return m_nranks; }
    uint32_t rank() { return m_rank; }

    /** Connect to the rendezvous server at master_ip:port, then set the backend up. */
    Status init(const char* master_ip, int port);
    /** Set the backend up with a caller-supplied broadcast instead of the server. */
    Status init(BcastCallback cb);

    Status send(const void* sendbuff, size_t len, DType dtype, uint32_t rank,
                std::shared_ptr<Context> ctx);
    Status recv(void* recvbuf, size_t len, DType dtype, uint32_t rank,
                std::shared_ptr<Context> ctx);

    virtual Status do_init() = 0;
    virtual Status do_init(BcastCallback cb) = 0;

    virtual Status scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                           uint32_t root, std::shared_ptr<Context> ctx) = 0;
    virtual Status gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                          uint32_t root, std::shared_ptr<Context> ctx) = 0;
    virtual Status all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                              std::shared_ptr<Context> ctx) = 0;
    virtual Status all_gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                              std::shared_ptr<Context> ctx) = 0;
    virtual Status all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                              ReduceOp op, std::shared_ptr<Context> ctx) = 0;
    virtual Status reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen,
                                  DType dtype, ReduceOp op, std::shared_ptr<Context> ctx) = 0;
    virtual Status broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                             uint32_t root, std::shared_ptr<Context> ctx) = 0;
    virtual Status reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                          ReduceOp op, uint32_t root, std::shared_ptr<Context> ctx) = 0;

    /** Bracket a series of send/recv so that they are issued together. */
    virtual Status group_start() = 0;
    virtual Status group_end() = 0;

    /** Which backend this is. */
    virtual Backend backend() const = 0;

    /** Make every later call fail with MEGRAY_ABORTED and release waits where possible. */
    virtual void abort() { m_aborted.store(true); }
    /** MEGRAY_OK, MEGRAY_ABORTED, or the first asynchronous failure seen (e.g. a device timeout). */
    virtual Status status() { return m_aborted.load() ? MEGRAY_ABORTED : MEGRAY_OK; }
    /** Snapshot of the activity counters. */
    virtual CommStats stats() { return m_stats; }

protected:
    uint32_t m_nranks;
    uint32_t m_rank;
    std::shared_ptr<Client> m_client;
    std::atomic<bool> m_aborted{false};
    CommStats m_stats;

    virtual Status _send(const void* sendbuff, size_t size, uint32_t rank,
                         std::shared_ptr<Context> ctx) = 0;
    virtual Status _recv(void* recvbuf, size_t size, uint32_t rank,
                         std::shared_ptr<Context> ctx) = 0;
};

}  // namespace MegRay
