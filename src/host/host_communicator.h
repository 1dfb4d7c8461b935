// Host backend (Backend MEGRAY_SHM): CPU ranks on one machine, as threads of
// one process or as separate processes.  Needs no GPU and makes no CUDA call
// when used with a HostContext; with a CudaContext, device buffers are staged
// through pinned host memory (as the reference's shm backend does,
// src/shm/all_reduce.cpp:88-124) and the call completes before it returns.
//
// Every collective is a sequence of "publish a piece into my slot / barrier /
// read the slots I need / barrier" steps over SharedRegion; reductions combine
// the ranks' data in rank order with cpu_reduce_n, for all ten numeric dtypes
// (the reference's host reduction lacks uint64, fp16 and fp64:
// src/shm/utils.cpp:41-68).  send/recv use one ring mailbox per ordered pair;
// between group_start and group_end they are queued and then progressed
// together, so that crossing sends cannot block each other.
#pragma once
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "host/shared_region.h"
#include "megray/communicator.h"

namespace MegRay {

class HostCommunicator : public Communicator {
public:
    HostCommunicator(uint32_t nranks, uint32_t rank);
    ~HostCommunicator() override;

    Status do_init() override;
    Status do_init(BcastCallback cb) override;

    Status scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype, uint32_t root,
                   std::shared_ptr<Context> ctx) override;
    Status gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype, uint32_t root,
                  std::shared_ptr<Context> ctx) override;
    Status all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                      std::shared_ptr<Context> ctx) override;
    Status all_gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                      std::shared_ptr<Context> ctx) override;
    Status all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype, ReduceOp op,
                      std::shared_ptr<Context> ctx) override;
    Status reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                          ReduceOp op, std::shared_ptr<Context> ctx) override;
    Status broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype, uint32_t root,
                     std::shared_ptr<Context> ctx) override;
    Status reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype, ReduceOp op,
                  uint32_t root, std::shared_ptr<Context> ctx) override;
    Status group_start() override;
    Status group_end() override;

    Backend backend() const override { return MEGRAY_SHM; }
    void abort() override;
    Status status() override;

    /** Barrier over the shared region (exposed for tests of the timeout path). */
    Status barrier();
    void set_timeout_ms(int64_t ms) { m_timeout_ms = ms; }

protected:
    Status _send(const void* sendbuff, size_t size, uint32_t rank,
                 std::shared_ptr<Context> ctx) override;
    Status _recv(void* recvbuf, size_t size, uint32_t rank, std::shared_ptr<Context> ctx) override;

private:
    struct P2POp {
        bool is_send;
        uint32_t peer;
        char* host;    // host pointer the bytes move through
        size_t bytes;
        size_t done;
        void* device;  // non-null: recv target on the device to fill afterwards
        std::shared_ptr<Context> ctx;
        std::shared_ptr<std::vector<char>> staging;
    };

    using Body = std::function<Status(const char* in, char* out)>;
    Status setup(const std::function<Status(char*, size_t)>& bcast, bool may_share_heap);
    Status check_ready(const std::shared_ptr<Context>& ctx) const;
    // Runs body on host-visible input/output (staging device buffers when ctx is CUDA).
    Status run(const std::shared_ptr<Context>& ctx, const void* in, size_t in_bytes, void* out,
               size_t out_bytes, const Body& body);
    Status sync_step() { return m_region->barrier(&m_sense, m_timeout_ms); }
    Status progress(std::vector<P2POp>& ops);
    Status fail(Status s);

    std::shared_ptr<host::SharedRegion> m_region;
    uint32_t m_sense = 0;
    int64_t m_timeout_ms;
    bool m_grouping = false;
    std::vector<P2POp> m_queued;
    Status m_error = MEGRAY_OK;
    void* m_pinned = nullptr;  // staging for CUDA contexts (grow-only)
    size_t m_pinned_bytes = 0;

    // CUDA contexts, stream-ordered: a call enqueues (1) the copy of its input into a pinned
    // staging slot, (2) a host function that hands the job to this communicator's worker thread
    // and returns at once, (3) a stream wait on a pinned word that the worker sets when the job is
    // done, (4) the copy of the result to the device; the caller never blocks.  The worker runs the
    // jobs in order (the barriers inside a job wait for the other ranks' workers, with the host
    // time limit).  The same semantics as the reference's shared-memory all_reduce (stream
    // callbacks around a CPU reducer thread, reference src/shm/all_reduce.cpp:88-124), without
    // callbacks that spin.
    struct AsyncState;
    AsyncState* m_async = nullptr;
    bool m_async_tried = false;
    Status run_stream_ordered(void* stream, const void* in, size_t in_bytes, void* out, size_t out_bytes,
                              const Body& body);
    void drain_async();  // wait until the worker has finished everything handed to it
    friend struct AsyncState;
};

}  // namespace MegRay
