// C-linkage doorway to the UNMODIFIED reference library (MegRay, compiled from its own
// sources by baseline/build_ref.py) so that Python can drive its public interface:
// create_server, get_communicator(MEGRAY_NCCL), Communicator::init and the collectives.
// Nothing of the new library is compiled or linked into this object.
#include <cuda_runtime.h>

#include <memory>

#include "megray.h"

namespace {
struct Box {
    std::shared_ptr<MegRay::Communicator> comm;
};
std::shared_ptr<MegRay::Context> ctx(void* stream) {
    return MegRay::CudaContext::make(static_cast<cudaStream_t>(stream));
}
}  // namespace

extern "C" {
int ref_get_free_port() { return MegRay::get_free_port(); }
int ref_create_server(unsigned nranks, int port) { return MegRay::create_server(nranks, port); }
void* ref_comm_new(unsigned nranks, unsigned rank) {
    try {
        auto* b = new Box;
        b->comm = MegRay::get_communicator(nranks, rank, MegRay::MEGRAY_NCCL);
        return b;
    } catch (...) {
        return nullptr;
    }
}
int ref_comm_init(void* c, const char* ip, int port) {
    try {
        return static_cast<Box*>(c)->comm->init(ip, port);
    } catch (...) {
        return -1;
    }
}
void ref_comm_delete(void* c) { delete static_cast<Box*>(c); }
int ref_all_gather(void* c, const void* s, void* r, size_t n, int dt, void* st) {
    return static_cast<Box*>(c)->comm->all_gather(s, r, n, static_cast<MegRay::DType>(dt), ctx(st));
}
int ref_reduce_scatter(void* c, const void* s, void* r, size_t n, int dt, int op, void* st) {
    return static_cast<Box*>(c)->comm->reduce_scatter(s, r, n, static_cast<MegRay::DType>(dt),
                                                      static_cast<MegRay::ReduceOp>(op), ctx(st));
}
int ref_all_reduce(void* c, const void* s, void* r, size_t n, int dt, int op, void* st) {
    return static_cast<Box*>(c)->comm->all_reduce(s, r, n, static_cast<MegRay::DType>(dt),
                                                  static_cast<MegRay::ReduceOp>(op), ctx(st));
}
int ref_all_to_all(void* c, const void* s, void* r, size_t n, int dt, void* st) {
    return static_cast<Box*>(c)->comm->all_to_all(s, r, n, static_cast<MegRay::DType>(dt), ctx(st));
}
int ref_broadcast(void* c, const void* s, void* r, size_t n, int dt, unsigned root, void* st) {
    return static_cast<Box*>(c)->comm->broadcast(s, r, n, static_cast<MegRay::DType>(dt), root, ctx(st));
}
int ref_reduce(void* c, const void* s, void* r, size_t n, int dt, int op, unsigned root, void* st) {
    return static_cast<Box*>(c)->comm->reduce(s, r, n, static_cast<MegRay::DType>(dt),
                                              static_cast<MegRay::ReduceOp>(op), root, ctx(st));
}
int ref_gather(void* c, const void* s, void* r, size_t n, int dt, unsigned root, void* st) {
    return static_cast<Box*>(c)->comm->gather(s, r, n, static_cast<MegRay::DType>(dt), root, ctx(st));
}
int ref_scatter(void* c, const void* s, void* r, size_t n, int dt, unsigned root, void* st) {
    return static_cast<Box*>(c)->comm->scatter(s, r, n, static_cast<MegRay::DType>(dt), root, ctx(st));
}
}
