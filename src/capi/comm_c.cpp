// C entry points for rendezvous, communicators, the NVL extras and the host
// oracle (see include/megray/c_api.h).  Exceptions never cross this boundary:
// they are logged and turned into a status.
#include <string.h>

#include "host/cpu_reduce.h"
#include "host/schedule_oracle.h"
#include "host/host_communicator.h"
#include "kernels/collectives.cuh"
#include "megray.h"
#include "megray/c_api.h"
#include "megray/trace.h"

using namespace MegRay;

namespace {

struct CommBox {
    std::shared_ptr<Communicator> comm;
};

std::shared_ptr<Context> make_ctx(int ctx_type, void* stream) {
    if (ctx_type == 0)
        return HostContext::make();
    return CudaContext::make(static_cast<cudaStream_t>(stream));
}

template <typename F>
int guarded(F&& f) {
    try {
        return static_cast<int>(f());
    } catch (const std::exception& e) {
        MEGRAY_ERROR("exception: %s", e.what());
        return MEGRAY_UNEXPECTED_ERR;
    }
}

Communicator* C(void* p) { return static_cast<CommBox*>(p)->comm.get(); }

}  // namespace

extern "C" {

int megray_get_host_ip(char* buf, size_t buflen) {
    char* ip = get_host_ip();
    if (ip == nullptr || buf == nullptr || buflen == 0) {
        delete[] ip;
        return 1;
    }
    snprintf(buf, buflen, "%s", ip);
    delete[] ip;
    return 0;
}
int megray_get_free_port(void) { return get_free_port(); }
int megray_create_server(uint32_t nranks, int port) {
    return guarded([&] { return create_server(nranks, port); });
}
void* megray_server_new(uint32_t nranks, int port) {
    try {
        return new Server(nranks, port);
    } catch (const std::exception& e) {
        MEGRAY_ERROR("server: %s", e.what());
        return nullptr;
    }
}
int megray_server_port(void* s) { return static_cast<Server*>(s)->port(); }
int megray_server_running(void* s) { return static_cast<Server*>(s)->running() ? 1 : 0; }
int megray_server_status(void* s) { return static_cast<Server*>(s)->status(); }
uint64_t megray_server_requests(void* s) { return static_cast<Server*>(s)->requests_served(); }
void megray_server_stop(void* s) { static_cast<Server*>(s)->stop(); }
void megray_server_delete(void* s) { delete static_cast<Server*>(s); }

void* megray_client_new(uint32_t nranks, uint32_t rank) { return new Client(nranks, rank); }
void megray_client_set_timeout_ms(void* c, int64_t ms) { static_cast<Client*>(c)->set_timeout_ms(ms); }
int megray_client_connect(void* c, const char* ip, int port) {
    return static_cast<Client*>(c)->connect(ip, port);
}
int megray_client_barrier(void* c) { return static_cast<Client*>(c)->barrier(); }
int megray_client_broadcast(void* c, const void* send, void* recv, size_t len, uint32_t root) {
    return static_cast<Client*>(c)->broadcast(send, recv, len, root);
}
int megray_client_allgather(void* c, const void* send, void* recv, size_t len) {
    return static_cast<Client*>(c)->allgather(send, recv, len);
}
void megray_client_delete(void* c) { delete static_cast<Client*>(c); }

void* megray_comm_new(uint32_t nranks, uint32_t rank, int backend) {
    try {
        auto* box = new CommBox;
        box->comm = get_communicator(nranks, rank, static_cast<Backend>(backend));
        return box;
    } catch (const std::exception& e) {
        MEGRAY_ERROR("get_communicator: %s", e.what());
        return nullptr;
    }
}
void megray_comm_delete(void* comm) { delete static_cast<CommBox*>(comm); }
int megray_comm_init(void* comm, const char* ip, int port) {
    return guarded([&] { return C(comm)->init(ip, port); });
}
int megray_comm_backend(void* comm) { return C(comm)->backend(); }
int megray_comm_status(void* comm) { return C(comm)->status(); }
void megray_comm_abort(void* comm) { C(comm)->abort(); }
void megray_comm_stats(void* comm, uint64_t* out) {
    CommStats s = C(comm)->stats();
    out[0] = s.calls;
    out[1] = s.bytes;
    out[2] = s.kernels;
    out[3] = s.timeouts;
    out[4] = s.algo_oneshot;
    out[5] = s.algo_twoshot;
    out[6] = s.algo_nvls;
    out[7] = s.algo_copy;
    out[8] = s.algo_ll;
    out[9] = s.algo_direct;
}

int megray_send(void* comm, const void* buf, size_t len, int dtype, uint32_t peer, int ct, void* st) {
    return guarded([&] { return C(comm)->send(buf, len, static_cast<DType>(dtype), peer, make_ctx(ct, st)); });
}
int megray_recv(void* comm, void* buf, size_t len, int dtype, uint32_t peer, int ct, void* st) {
    return guarded([&] { return C(comm)->recv(buf, len, static_cast<DType>(dtype), peer, make_ctx(ct, st)); });
}
int megray_scatter(void* comm, const void* send, void* recv, size_t recvlen, int dtype, uint32_t root, int ct, void* st) {
    return guarded([&] { return C(comm)->scatter(send, recv, recvlen, static_cast<DType>(dtype), root, make_ctx(ct, st)); });
}
int megray_gather(void* comm, const void* send, void* recv, size_t sendlen, int dtype, uint32_t root, int ct, void* st) {
    return guarded([&] { return C(comm)->gather(send, recv, sendlen, static_cast<DType>(dtype), root, make_ctx(ct, st)); });
}
int megray_all_to_all(void* comm, const void* send, void* recv, size_t len, int dtype, int ct, void* st) {
    return guarded([&] { return C(comm)->all_to_all(send, recv, len, static_cast<DType>(dtype), make_ctx(ct, st)); });
}
int megray_all_gather(void* comm, const void* send, void* recv, size_t sendlen, int dtype, int ct, void* st) {
    return guarded([&] { return C(comm)->all_gather(send, recv, sendlen, static_cast<DType>(dtype), make_ctx(ct, st)); });
}
int megray_all_reduce(void* comm, const void* send, void* recv, size_t len, int dtype, int op, int ct, void* st) {
    return guarded([&] {
        return C(comm)->all_reduce(send, recv, len, static_cast<DType>(dtype), static_cast<ReduceOp>(op), make_ctx(ct, st));
    });
}
int megray_reduce_scatter(void* comm, const void* send, void* recv, size_t recvlen, int dtype, int op, int ct, void* st) {
    return guarded([&] {
        return C(comm)->reduce_scatter(send, recv, recvlen, static_cast<DType>(dtype), static_cast<ReduceOp>(op), make_ctx(ct, st));
    });
}
int megray_broadcast(void* comm, const void* send, void* recv, size_t len, int dtype, uint32_t root, int ct, void* st) {
    return guarded([&] { return C(comm)->broadcast(send, recv, len, static_cast<DType>(dtype), root, make_ctx(ct, st)); });
}
int megray_reduce(void* comm, const void* send, void* recv, size_t len, int dtype, int op, uint32_t root, int ct, void* st) {
    return guarded([&] {
        return C(comm)->reduce(send, recv, len, static_cast<DType>(dtype), static_cast<ReduceOp>(op), root, make_ctx(ct, st));
    });
}
int megray_group_start(void* comm) { return guarded([&] { return C(comm)->group_start(); }); }
int megray_group_end(void* comm) { return guarded([&] { return C(comm)->group_end(); }); }
int megray_host_barrier(void* comm) {
    auto* h = dynamic_cast<HostCommunicator*>(C(comm));
    return h ? h->barrier() : MEGRAY_INVALID_USAGE;
}
void megray_host_set_timeout_ms(void* comm, int64_t ms) {
    auto* h = dynamic_cast<HostCommunicator*>(C(comm));
    if (h)
        h->set_timeout_ms(ms);
}

void* megray_nvl_alloc(void* comm, size_t bytes, size_t* offset_out) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->sym_alloc(bytes, offset_out) : nullptr;
}
int megray_nvl_free(void* comm, void* ptr) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->sym_free(ptr) : MEGRAY_INVALID_USAGE;
}
void* megray_nvl_peer_ptr(void* comm, void* ptr, uint32_t peer) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->peer_ptr(ptr, peer) : nullptr;
}
int megray_nvl_register(void* comm, void* ptr, size_t bytes) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->register_buffer(ptr, bytes) : MEGRAY_INVALID_USAGE;
}
int megray_nvl_deregister(void* comm, void* ptr) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->deregister_buffer(ptr) : MEGRAY_INVALID_USAGE;
}
void* megray_nvl_heap_base(void* comm, uint32_t peer) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->heap_base(peer) : nullptr;
}
size_t megray_nvl_heap_bytes(void* comm) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->heap_bytes() : 0;
}
int megray_nvl_all_reduce_scaled(void* comm, const void* send, void* recv, size_t len, int in_dtype,
                                 int out_dtype, float scale, int op, void* stream) {
    NvlInterface* n = as_nvl(C(comm));
    if (!n)
        return MEGRAY_INVALID_USAGE;
    return guarded([&] {
        return n->all_reduce_scaled(send, recv, len, static_cast<DType>(in_dtype), static_cast<DType>(out_dtype),
                                    scale, static_cast<ReduceOp>(op), make_ctx(1, stream));
    });
}
int megray_nvl_stream_barrier(void* comm, void* stream) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->stream_barrier(make_ctx(1, stream)) : MEGRAY_INVALID_USAGE;
}
void megray_nvl_set_device_timeout_ms(void* comm, int64_t ms) {
    NvlInterface* n = as_nvl(C(comm));
    if (n)
        n->set_device_timeout_ms(ms);
}
int megray_nvl_check_canaries(void* comm) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->check_canaries() : MEGRAY_INVALID_USAGE;
}
void megray_nvl_set_p2p_async(void* comm, int on) {
    NvlInterface* n = as_nvl(C(comm));
    if (n)
        n->set_p2p_async(on != 0);
}
int megray_nvl_p2p_join(void* comm, void* stream) {
    NvlInterface* n = as_nvl(C(comm));
    return n ? n->p2p_join(make_ctx(1, stream)) : MEGRAY_INVALID_USAGE;
}

int megray_cpu_reduce_n(const void* const* in, int n_in, void* out, size_t len, int dtype, int op) {
    return host::cpu_reduce_n(in, n_in, out, len, static_cast<DType>(dtype), static_cast<ReduceOp>(op));
}
int megray_oracle_ring_all_reduce(const void* const* in, void* const* out, int nranks, size_t len, int dtype,
                                  int op) {
    return host::ring_all_reduce_schedule(in, out, nranks, len, static_cast<DType>(dtype),
                                          static_cast<ReduceOp>(op));
}
int megray_oracle_tree_reduce(const void* const* in, void* out, int nranks, int root, size_t len, int dtype,
                              int op) {
    return host::tree_reduce_schedule(in, out, nranks, root, len, static_cast<DType>(dtype),
                                      static_cast<ReduceOp>(op));
}
int megray_cpu_reduce_scale_cast(const void* const* in, int n_in, int in_dtype, void* out, int out_dtype,
                                 size_t len, int op, double scale) {
    return host::cpu_reduce_scale_cast(in, n_in, static_cast<DType>(in_dtype), out, static_cast<DType>(out_dtype),
                                       len, static_cast<ReduceOp>(op), scale);
}
int megray_reduce_n(const void* const* in, int n_in, void* out, size_t len, int in_dtype, int out_dtype,
                    int op, float scale, void* stream) {
    cudaError_t e = mgk::coll::launch_reduce_n(in, n_in, out, len, static_cast<DType>(in_dtype),
                                               static_cast<DType>(out_dtype), static_cast<ReduceOp>(op), scale,
                                               static_cast<cudaStream_t>(stream));
    return e == cudaSuccess ? 0 : -static_cast<int>(e);
}

size_t megray_dtype_size(int dtype) {
    if (dtype < 0 || dtype >= MEGRAY_DTYPE_COUNT)
        return 0;
    return get_dtype_size(static_cast<DType>(dtype));
}
void megray_set_log_level(int level) { set_log_level(level); }
void megray_trace_enable(const char* path) { trace_enable(path); }
size_t megray_trace_dump(void) { return trace_dump(); }

}  // extern "C"
