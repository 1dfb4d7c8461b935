// NCCL backend (Backend MEGRAY_NCCL): each call maps to the one matching NCCL
// call on the context's stream, as in the reference backend
// (src/nccl/communicator.cpp:66-240).  It is the baseline the native NVLink
// backend is measured against, and the send/recv engine that backend reuses.
//
// Differences from the reference wrapper: bf16 is mapped; the
// NCCL_LAUNCH_MODE=PARALLEL gate on scatter/gather/all_to_all
// (src/nccl/communicator.cpp:20-27) is dropped, because NCCL >= 2.18 no longer
// needs it for grouped calls issued from one thread per rank; abort() ends a
// stuck communicator with ncclCommAbort and status() reports asynchronous
// NCCL errors.
#pragma once
#include <memory>

#include "megray/communicator.h"

namespace MegRay {

struct NcclCommunicatorPrivate;

class NcclCommunicator : public Communicator {
public:
    NcclCommunicator(uint32_t nranks, uint32_t rank);
    ~NcclCommunicator() override;

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

    Backend backend() const override { return MEGRAY_NCCL; }
    void abort() override;
    Status status() override;

    /** Bytes of the bootstrap blob (the NCCL unique id) that init broadcasts. */
    static size_t unique_id_bytes();

protected:
    Status _send(const void* sendbuff, size_t size, uint32_t rank,
                 std::shared_ptr<Context> ctx) override;
    Status _recv(void* recvbuf, size_t size, uint32_t rank, std::shared_ptr<Context> ctx) override;

private:
    Status finish_init(void* uid);
    std::unique_ptr<NcclCommunicatorPrivate> m_nccl;
};

}  // namespace MegRay
