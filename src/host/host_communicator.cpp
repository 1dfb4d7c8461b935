#include "host/host_communicator.h"
#include "megray/trace.h"

#include <sched.h>
#include <string.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>

#include "host/cpu_reduce.h"
#include "megray/options.h"

#ifdef MEGRAY_WITH_CUDA
#include <cuda.h>
#include <cuda_runtime_api.h>

#include "megray/cuda_context.h"
#endif

namespace MegRay {

namespace {

struct Hello {
    char name[64];
    int32_t pid;
    int32_t in_process;
    uint64_t slot_bytes;
    uint64_t mailbox_bytes;
};

int64_t now_ms() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

std::atomic<uint32_t> g_group_counter{0};

size_t env_kb(const char* name, size_t dflt_kb) {
    const char* e = getenv(name);
    if (e == nullptr || *e == 0)
        return dflt_kb << 10;
    long long v = atoll(e);
    return v > 0 ? static_cast<size_t>(v) << 10 : dflt_kb << 10;
}

}  // namespace

#ifdef MEGRAY_WITH_CUDA
// Everything the stream-ordered path of one communicator owns.
struct HostCommunicator::AsyncState {
    struct Job {
        AsyncState* owner;
        std::function<Status()> work;
        uint32_t seq;
    };
    struct Slot {
        void* pinned = nullptr;
        size_t bytes = 0;
        cudaEvent_t done = nullptr;  // recorded after the slot's result left for the device
        bool used = false;
    };
    static constexpr int kSlots = 4;
    using WaitValueFn = CUresult (*)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);

    HostCommunicator* comm;
    WaitValueFn wait_value = nullptr;
    volatile uint32_t* done_host = nullptr;  // pinned, mapped: number of the last finished job
    CUdeviceptr done_dev = 0;
    uint32_t next_seq = 0;
    Slot slots[kSlots];
    int next_slot = 0;
    std::vector<cudaStream_t> streams;  // every stream a job was enqueued on
    std::mutex mu;
    std::condition_variable cv, idle_cv;
    std::deque<Job*> queue;
    bool busy = false, stop = false;
    std::atomic<int> error{0};
    std::thread worker;

    explicit AsyncState(HostCommunicator* c) : comm(c) {}

    bool start() {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess || fn == nullptr) {
            (void)cudaGetLastError();
            return false;
        }
        wait_value = reinterpret_cast<WaitValueFn>(fn);
        void* h = nullptr;
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped) != cudaSuccess) {
            (void)cudaGetLastError();
            return false;
        }
        memset(h, 0, 64);
        void* d = nullptr;
        if (cudaHostGetDevicePointer(&d, h, 0) != cudaSuccess) {
            (void)cudaGetLastError();
            cudaFreeHost(h);
            return false;
        }
        done_host = static_cast<volatile uint32_t*>(h);
        done_dev = reinterpret_cast<CUdeviceptr>(d);
        worker = std::thread([this] { loop(); });
        return true;
    }

    void loop() {
        for (;;) {
            Job* job = nullptr;
            {
                std::unique_lock<std::mutex> lk(mu);
                cv.wait(lk, [&] { return stop || !queue.empty(); });
                if (queue.empty())
                    return;
                job = queue.front();
                queue.pop_front();
                busy = true;
            }
            const Status s = job->work();
            if (s != MEGRAY_OK) {
                int expected = 0;
                error.compare_exchange_strong(expected, static_cast<int>(s));
            }
            // the stream that waits for this job goes on, whatever the outcome
            __atomic_store_n(const_cast<uint32_t*>(done_host), job->seq, __ATOMIC_RELEASE);
            delete job;
            {
                std::lock_guard<std::mutex> lk(mu);
                busy = false;
            }
            idle_cv.notify_all();
        }
    }

    static void CUDART_CB hand_over(void* p) {  // runs on a driver thread: must not block
        Job* job = static_cast<Job*>(p);
        AsyncState* a = job->owner;
        {
            std::lock_guard<std::mutex> lk(a->mu);
            a->queue.push_back(job);
        }
        a->cv.notify_one();
    }

    void drain() {
        std::unique_lock<std::mutex> lk(mu);
        idle_cv.wait(lk, [&] { return queue.empty() && !busy; });
    }

    ~AsyncState() {
        for (cudaStream_t s : streams)
            cudaStreamSynchronize(s);  // every job has been handed over and waited for
        {
            std::lock_guard<std::mutex> lk(mu);
            stop = true;
        }
        cv.notify_all();
        if (worker.joinable())
            worker.join();
        for (Slot& sl : slots) {
            if (sl.done != nullptr)
                cudaEventDestroy(sl.done);
            if (sl.pinned != nullptr)
                cudaFreeHost(sl.pinned);
        }
        if (done_host != nullptr)
            cudaFreeHost(const_cast<uint32_t*>(done_host));
    }
};
#else
struct HostCommunicator::AsyncState {};
#endif

HostCommunicator::HostCommunicator(uint32_t nranks, uint32_t rank) : Communicator(nranks, rank) {
    m_timeout_ms = global_options().timeout_ms;
}

HostCommunicator::~HostCommunicator() {
#ifdef MEGRAY_WITH_CUDA
    delete m_async;
    if (m_pinned != nullptr)
        cudaFreeHost(m_pinned);
#endif
}

void HostCommunicator::drain_async() {
#ifdef MEGRAY_WITH_CUDA
    if (m_async != nullptr) {
        for (cudaStream_t s : m_async->streams)
            cudaStreamSynchronize(s);
        m_async->drain();
        const int e = m_async->error.load();
        if (e != 0)
            fail(static_cast<Status>(e));
    }
#endif
}

Status HostCommunicator::run_stream_ordered(void* stream_v, const void* in, size_t in_bytes, void* out,
                                            size_t out_bytes, const Body& body) {
#ifdef MEGRAY_WITH_CUDA
    cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
    AsyncState& a = *m_async;
    const int e = a.error.load();
    if (e != 0)
        return fail(static_cast<Status>(e));
    AsyncState::Slot& sl = a.slots[a.next_slot];
    a.next_slot = (a.next_slot + 1) % AsyncState::kSlots;
    if (sl.used)
        CUDA_CHECK(cudaEventSynchronize(sl.done));  // (blocks only when four calls are in flight)
    const size_t need = in_bytes + out_bytes;
    if (need > sl.bytes) {
        if (sl.pinned != nullptr)
            cudaFreeHost(sl.pinned);
        sl.pinned = nullptr;
        sl.bytes = 0;
        CUDA_CHECK(cudaHostAlloc(&sl.pinned, std::max<size_t>(need, 4096), cudaHostAllocDefault));
        sl.bytes = std::max<size_t>(need, 4096);
    }
    if (sl.done == nullptr)
        CUDA_CHECK(cudaEventCreateWithFlags(&sl.done, cudaEventDisableTiming));
    char* h_in = static_cast<char*>(sl.pinned);
    char* h_out = h_in + in_bytes;
    if (std::find(a.streams.begin(), a.streams.end(), stream) == a.streams.end())
        a.streams.push_back(stream);
    if (in_bytes)
        CUDA_CHECK(cudaMemcpyAsync(h_in, in, in_bytes, cudaMemcpyDeviceToHost, stream));
    auto* job = new AsyncState::Job;
    job->owner = &a;
    job->seq = ++a.next_seq;
    const char* hin = in_bytes ? h_in : nullptr;
    char* hout = out_bytes ? h_out : nullptr;
    job->work = [body, hin, hout] { return body(hin, hout); };
    cudaError_t ce = cudaLaunchHostFunc(stream, AsyncState::hand_over, job);
    if (ce != cudaSuccess) {
        delete job;
        CUDA_CHECK(ce);
    }
    if (a.wait_value(stream, a.done_dev, job->seq, CU_STREAM_WAIT_VALUE_GEQ) != CUDA_SUCCESS) {
        // the job is on its way: wait for it the blocking way
        CUDA_CHECK(cudaStreamSynchronize(stream));
        a.drain();
    }
    if (out_bytes)
        CUDA_CHECK(cudaMemcpyAsync(out, h_out, out_bytes, cudaMemcpyHostToDevice, stream));
    CUDA_CHECK(cudaEventRecord(sl.done, stream));
    sl.used = true;
    return MEGRAY_OK;
#else
    (void)stream_v; (void)in; (void)in_bytes; (void)out; (void)out_bytes; (void)body;
    return MEGRAY_INVALID_ARGUMENT;
#endif
}

Status HostCommunicator::fail(Status s) {
    if (s != MEGRAY_OK && m_error == MEGRAY_OK)
        m_error = s;
    if (s == MEGRAY_TIMEOUT)
        m_stats.timeouts++;
    return s;
}

void HostCommunicator::abort() {
    Communicator::abort();
    if (m_region)
        m_region->abort();
}

Status HostCommunicator::status() {
#ifdef MEGRAY_WITH_CUDA
    if (m_async != nullptr && m_error == MEGRAY_OK) {
        const int e = m_async->error.load();
        if (e != 0)
            fail(static_cast<Status>(e));
    }
#endif
    if (m_aborted.load() || (m_region && m_region->aborted()))
        return m_error != MEGRAY_OK ? m_error : MEGRAY_ABORTED;
    return m_error;
}

Status HostCommunicator::do_init() {
    // With the rendezvous client we can find out whether all ranks share one
    // process (then a heap block is shared) before rank 0 creates the region.
    std::vector<int32_t> pids(m_nranks);
    int32_t me = static_cast<int32_t>(getpid());
    MEGRAY_CHECK(m_client->allgather(&me, pids.data(), sizeof(me)));
    bool same = true;
    for (uint32_t r = 0; r < m_nranks; ++r)
        same = same && pids[r] == pids[0];
    auto bcast = [this](char* buf, size_t len) { return m_client->broadcast(buf, buf, len, 0); };
    MEGRAY_CHECK(setup(bcast, same));
    return m_client->barrier();
}

Status HostCommunicator::do_init(BcastCallback cb) {
    auto bcast = [&cb](char* buf, size_t len) {
        cb(buf, len);
        return MEGRAY_OK;
    };
    return setup(bcast, false);
}

Status HostCommunicator::setup(const std::function<Status(char*, size_t)>& bcast,
                               bool may_share_heap) {
    Hello h;
    memset(&h, 0, sizeof(h));
    if (m_rank == 0) {
        snprintf(h.name, sizeof(h.name), "/megray_%d_%u_%llx", static_cast<int>(getpid()),
                 g_group_counter.fetch_add(1), static_cast<unsigned long long>(now_ms()));
        h.pid = static_cast<int32_t>(getpid());
        h.in_process = may_share_heap ? 1 : 0;
        h.slot_bytes = env_kb("MEGRAY_HOST_SLOT_KB", 4096);
        h.mailbox_bytes = env_kb("MEGRAY_HOST_MAILBOX_KB", 256);
        m_region = host::SharedRegion::create(h.name, m_nranks, h.slot_bytes, h.mailbox_bytes,
                                              h.in_process != 0);
        if (!m_region)
            return MEGRAY_SYS_ERROR;
    }
    MEGRAY_CHECK(bcast(reinterpret_cast<char*>(&h), sizeof(h)));
    if (m_rank != 0) {
        h.name[sizeof(h.name) - 1] = 0;
        m_region = host::SharedRegion::attach(h.name, h.in_process != 0,
                                              global_options().connect_timeout_ms);
        if (!m_region)
            return MEGRAY_SYS_ERROR;
        if (m_region->nranks() != m_nranks) {
            MEGRAY_ERROR("shared region is for %u ranks, this group has %u", m_region->nranks(),
                         m_nranks);
            return MEGRAY_INVALID_USAGE;
        }
    }
    // everybody attached before anyone starts using slots
    const int64_t t0 = now_ms();
    while (m_region->header()->attached.load() < m_nranks) {
        if (now_ms() - t0 > global_options().connect_timeout_ms)
            return fail(MEGRAY_TIMEOUT);
        sched_yield();
    }
    return MEGRAY_OK;
}

Status HostCommunicator::check_ready(const std::shared_ptr<Context>& ctx) const {
    if (!m_region) {
        MEGRAY_ERROR("communicator used before init");
        return MEGRAY_INVALID_USAGE;
    }
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    if (!ctx)
        return MEGRAY_INVALID_ARGUMENT;
    if (ctx->type() == MEGRAY_CTX_DEFAULT)
        return MEGRAY_OK;
#ifdef MEGRAY_WITH_CUDA
    if (ctx->type() == MEGRAY_CTX_CUDA)
        return MEGRAY_OK;
#endif
    MEGRAY_ERROR("host backend: unsupported context type %d", ctx->type());
    return MEGRAY_INVALID_ARGUMENT;
}

Status HostCommunicator::barrier() {
    if (!m_region)
        return MEGRAY_INVALID_USAGE;
    drain_async();
    return fail(sync_step());
}

Status HostCommunicator::run(const std::shared_ptr<Context>& ctx, const void* in, size_t in_bytes,
                             void* out, size_t out_bytes, const Body& body) {
    MEGRAY_CHECK(check_ready(ctx));
    m_stats.calls++;
    m_stats.bytes += std::max(in_bytes, out_bytes);
    if (ctx->type() == MEGRAY_CTX_DEFAULT) {
        drain_async();  // jobs of CUDA contexts use the same barrier state
        return fail(body(static_cast<const char*>(in), static_cast<char*>(out)));
    }
#ifdef MEGRAY_WITH_CUDA
    cudaStream_t stream = static_cast<CudaContext*>(ctx.get())->get_stream();
    if (in == nullptr)
        in_bytes = 0;
    if (out == nullptr)
        out_bytes = 0;
    if (m_async == nullptr && !m_async_tried) {
        m_async_tried = true;
        static const bool wanted = [] {
            const char* e = getenv("MEGRAY_HOST_STREAM_ORDERED");
            return e == nullptr || atoi(e) != 0;
        }();
        if (wanted) {
            m_async = new AsyncState(this);
            if (!m_async->start()) {
                delete m_async;
                m_async = nullptr;
            }
        }
    }
    if (m_async != nullptr)
        return run_stream_ordered(stream, in, in_bytes, out, out_bytes, body);
    const size_t need = in_bytes + out_bytes;
    if (need > m_pinned_bytes) {
        if (m_pinned != nullptr)
            cudaFreeHost(m_pinned);
        m_pinned = nullptr;
        m_pinned_bytes = 0;
        CUDA_CHECK(cudaHostAlloc(&m_pinned, need, cudaHostAllocDefault));
        m_pinned_bytes = need;
    }
    char* h_in = static_cast<char*>(m_pinned);
    char* h_out = h_in + in_bytes;
    if (in_bytes)
        CUDA_CHECK(cudaMemcpyAsync(h_in, in, in_bytes, cudaMemcpyDeviceToHost, stream));
    CUDA_CHECK(cudaStreamSynchronize(stream));
    Status s = body(in_bytes ? h_in : nullptr, out_bytes ? h_out : nullptr);
    if (s != MEGRAY_OK)
        return fail(s);
    if (out_bytes) {
        CUDA_CHECK(cudaMemcpyAsync(out, h_out, out_bytes, cudaMemcpyHostToDevice, stream));
        CUDA_CHECK(cudaStreamSynchronize(stream));
    }
    return MEGRAY_OK;
#else
    return MEGRAY_INVALID_ARGUMENT;
#endif
}

// ------------------------------------------------------------------ collectives
// In every loop below `piece` is a byte count that fits the slots, `off` the
// byte offset of the piece inside each rank's logical buffer.

Status HostCommunicator::all_gather(const void* sendbuff, void* recvbuff, size_t sendlen,
                                    DType dtype, std::shared_ptr<Context> ctx) {
    const size_t bytes = sendlen * get_dtype_size(dtype);
    TraceScope trace("all_gather", bytes, m_rank);
    return run(ctx, sendbuff, bytes, recvbuff, bytes * m_nranks, [=](const char* in, char* out) {
        const size_t cap = m_region->slot_bytes();
        for (size_t off = 0; off < bytes || off == 0; off += cap) {
            const size_t piece = std::min(cap, bytes - off);
            memcpy(m_region->slot(m_rank), in + off, piece);
            MEGRAY_CHECK(sync_step());
            for (uint32_t r = 0; r < m_nranks; ++r)
                memcpy(out + r * bytes + off, m_region->slot(r), piece);
            MEGRAY_CHECK(sync_step());
            if (bytes == 0)
                break;
        }
        return MEGRAY_OK;
    });
}

Status HostCommunicator::all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                    ReduceOp op, std::shared_ptr<Context> ctx) {
    if (dtype == MEGRAY_CHAR)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t esz = get_dtype_size(dtype);
    const size_t bytes = len * esz;
    TraceScope trace("all_reduce", bytes, m_rank);
    return run(ctx, sendbuff, bytes, recvbuff, bytes, [=](const char* in, char* out) {
        const size_t cap_elems = m_region->slot_bytes() / esz;
        std::vector<const void*> srcs(m_nranks);
        for (size_t e0 = 0; e0 < len || e0 == 0; e0 += cap_elems) {
            const size_t n = std::min(cap_elems, len - e0);
            memcpy(m_region->slot(m_rank), in + e0 * esz, n * esz);
            MEGRAY_CHECK(sync_step());
            // rank r reduces the r-th share of the piece into the result slot
            const size_t share = (n + m_nranks - 1) / m_nranks;
            const size_t b = std::min(n, share * m_rank), e = std::min(n, b + share);
            for (uint32_t r = 0; r < m_nranks; ++r)
                srcs[r] = m_region->slot(r) + b * esz;
            MEGRAY_CHECK(host::cpu_reduce_n(srcs.data(), static_cast<int>(m_nranks),
                                            m_region->result() + b * esz, e - b, dtype, op));
            MEGRAY_CHECK(sync_step());
            memcpy(out + e0 * esz, m_region->result(), n * esz);
            MEGRAY_CHECK(sync_step());
            if (len == 0)
                break;
        }
        return MEGRAY_OK;
    });
}

Status HostCommunicator::reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen,
                                        DType dtype, ReduceOp op, std::shared_ptr<Context> ctx) {
    if (dtype == MEGRAY_CHAR)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t esz = get_dtype_size(dtype);
    const size_t bytes = recvlen * esz;
    TraceScope trace("reduce_scatter", bytes, m_rank);
    return run(ctx, sendbuff, bytes * m_nranks, recvbuff, bytes, [=](const char* in, char* out) {
        // each rank publishes, for every destination d, a piece of chunk d
        const size_t cap_elems = std::max<size_t>(1, m_region->slot_bytes() / m_nranks / esz);
        std::vector<const void*> srcs(m_nranks);
        for (size_t e0 = 0; e0 < recvlen || e0 == 0; e0 += cap_elems) {
            const size_t n = std::min(cap_elems, recvlen - e0);
            for (uint32_t d = 0; d < m_nranks; ++d)
                memcpy(m_region->slot(m_rank) + d * cap_elems * esz,
                       in + (d * recvlen + e0) * esz, n * esz);
            MEGRAY_CHECK(sync_step());
            for (uint32_t r = 0; r < m_nranks; ++r)
                srcs[r] = m_region->slot(r) + m_rank * cap_elems * esz;
            MEGRAY_CHECK(host::cpu_reduce_n(srcs.data(), static_cast<int>(m_nranks), out + e0 * esz,
                                            n, dtype, op));
            MEGRAY_CHECK(sync_step());
            if (recvlen == 0)
                break;
        }
        return MEGRAY_OK;
    });
}

Status HostCommunicator::all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                    std::shared_ptr<Context> ctx) {
    const size_t bytes = len * get_dtype_size(dtype);
    TraceScope trace("all_to_all", bytes, m_rank);
    return run(ctx, sendbuff, bytes * m_nranks, recvbuff, bytes * m_nranks,
               [=](const char* in, char* out) {
                   const size_t cap = std::max<size_t>(1, m_region->slot_bytes() / m_nranks);
                   for (size_t off = 0; off < bytes || off == 0; off += cap) {
                       const size_t piece = std::min(cap, bytes - off);
                       for (uint32_t d = 0; d < m_nranks; ++d)
                           memcpy(m_region->slot(m_rank) + d * cap, in + d * bytes + off, piece);
                       MEGRAY_CHECK(sync_step());
                       for (uint32_t r = 0; r < m_nranks; ++r)
                           memcpy(out + r * bytes + off, m_region->slot(r) + m_rank * cap, piece);
                       MEGRAY_CHECK(sync_step());
                       if (bytes == 0)
                           break;
                   }
                   return MEGRAY_OK;
               });
}

Status HostCommunicator::broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                   uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t bytes = len * get_dtype_size(dtype);
    TraceScope trace("broadcast", bytes, m_rank);
    const bool is_root = m_rank == root;
    return run(ctx, is_root ? sendbuff : nullptr, is_root ? bytes : 0, recvbuff, bytes,
               [=](const char* in, char* out) {
                   const size_t cap = m_region->slot_bytes();
                   for (size_t off = 0; off < bytes || off == 0; off += cap) {
                       const size_t piece = std::min(cap, bytes - off);
                       if (is_root)
                           memcpy(m_region->slot(root), in + off, piece);
                       MEGRAY_CHECK(sync_step());
                       memcpy(out + off, m_region->slot(root), piece);
                       MEGRAY_CHECK(sync_step());
                       if (bytes == 0)
                           break;
                   }
                   return MEGRAY_OK;
               });
}

Status HostCommunicator::reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                ReduceOp op, uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks || dtype == MEGRAY_CHAR)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t esz = get_dtype_size(dtype);
    const size_t bytes = len * esz;
    TraceScope trace("reduce", bytes, m_rank);
    const bool is_root = m_rank == root;
    return run(ctx, sendbuff, bytes, is_root ? recvbuff : nullptr, is_root ? bytes : 0,
               [=](const char* in, char* out) {
                   const size_t cap_elems = m_region->slot_bytes() / esz;
                   std::vector<const void*> srcs(m_nranks);
                   for (size_t e0 = 0; e0 < len || e0 == 0; e0 += cap_elems) {
                       const size_t n = std::min(cap_elems, len - e0);
                       memcpy(m_region->slot(m_rank), in + e0 * esz, n * esz);
                       MEGRAY_CHECK(sync_step());
                       if (is_root) {
                           for (uint32_t r = 0; r < m_nranks; ++r)
                               srcs[r] = m_region->slot(r);
                           MEGRAY_CHECK(host::cpu_reduce_n(srcs.data(), static_cast<int>(m_nranks),
                                                           out + e0 * esz, n, dtype, op));
                       }
                       MEGRAY_CHECK(sync_step());
                       if (len == 0)
                           break;
                   }
                   return MEGRAY_OK;
               });
}

Status HostCommunicator::gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                                uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t bytes = sendlen * get_dtype_size(dtype);
    TraceScope trace("gather", bytes, m_rank);
    const bool is_root = m_rank == root;
    return run(ctx, sendbuff, bytes, is_root ? recvbuff : nullptr, is_root ? bytes * m_nranks : 0,
               [=](const char* in, char* out) {
                   const size_t cap = m_region->slot_bytes();
                   for (size_t off = 0; off < bytes || off == 0; off += cap) {
                       const size_t piece = std::min(cap, bytes - off);
                       memcpy(m_region->slot(m_rank), in + off, piece);
                       MEGRAY_CHECK(sync_step());
                       if (is_root)
                           for (uint32_t r = 0; r < m_nranks; ++r)
                               memcpy(out + r * bytes + off, m_region->slot(r), piece);
                       MEGRAY_CHECK(sync_step());
                       if (bytes == 0)
                           break;
                   }
                   return MEGRAY_OK;
               });
}

Status HostCommunicator::scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                                 uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    const size_t bytes = recvlen * get_dtype_size(dtype);
    TraceScope trace("scatter", bytes, m_rank);
    const bool is_root = m_rank == root;
    return run(ctx, is_root ? sendbuff : nullptr, is_root ? bytes * m_nranks : 0, recvbuff, bytes,
               [=](const char* in, char* out) {
                   const size_t cap = std::max<size_t>(1, m_region->slot_bytes() / m_nranks);
                   for (size_t off = 0; off < bytes || off == 0; off += cap) {
                       const size_t piece = std::min(cap, bytes - off);
                       if (is_root)
                           for (uint32_t d = 0; d < m_nranks; ++d)
                               memcpy(m_region->slot(root) + d * cap, in + d * bytes + off, piece);
                       MEGRAY_CHECK(sync_step());
                       memcpy(out + off, m_region->slot(root) + m_rank * cap, piece);
                       MEGRAY_CHECK(sync_step());
                       if (bytes == 0)
                           break;
                   }
                   return MEGRAY_OK;
               });
}

// ------------------------------------------------------------------ send / recv

Status HostCommunicator::progress(std::vector<P2POp>& ops) {
    const size_t cap = m_region->mailbox_bytes();
    const int64_t t0 = now_ms();
    size_t open = ops.size();
    uint32_t idle = 0;
    while (open > 0) {
        bool moved = false;
        open = 0;
        // one byte stream per ordered pair: only the oldest unfinished op of a
        // (direction, peer) may move, so that queued messages do not interleave
        uint64_t busy_send = 0, busy_recv = 0;
        for (P2POp& op : ops) {
            if (op.done == op.bytes)
                continue;
            uint64_t& busy = op.is_send ? busy_send : busy_recv;
            const uint64_t bit = 1ull << (op.peer & 63);
            if (busy & bit) {
                ++open;
                continue;
            }
            busy |= bit;
            host::Mailbox* mb = op.is_send ? m_region->mailbox(m_rank, op.peer)
                                           : m_region->mailbox(op.peer, m_rank);
            char* ring = op.is_send ? m_region->mailbox_data(m_rank, op.peer)
                                    : m_region->mailbox_data(op.peer, m_rank);
            const uint64_t head = mb->head.load(std::memory_order_acquire);
            const uint64_t tail = mb->tail.load(std::memory_order_acquire);
            size_t room = op.is_send ? cap - static_cast<size_t>(head - tail)
                                     : static_cast<size_t>(head - tail);
            size_t n = std::min(room, op.bytes - op.done);
            if (n > 0) {
                const size_t pos = static_cast<size_t>((op.is_send ? head : tail) % cap);
                const size_t first = std::min(n, cap - pos);
                if (op.is_send) {
                    memcpy(ring + pos, op.host + op.done, first);
                    memcpy(ring, op.host + op.done + first, n - first);
                    mb->head.store(head + n, std::memory_order_release);
                } else {
                    memcpy(op.host + op.done, ring + pos, first);
                    memcpy(op.host + op.done + first, ring, n - first);
                    mb->tail.store(tail + n, std::memory_order_release);
                }
                op.done += n;
                moved = true;
            }
            if (op.done != op.bytes)
                ++open;
        }
        if (moved) {
            idle = 0;
            continue;
        }
        if (++idle > 200)
            sched_yield();
        if ((idle & 0xff) == 0) {
            if (m_region->aborted() || m_aborted.load())
                return MEGRAY_ABORTED;
            if (m_timeout_ms > 0 && now_ms() - t0 > m_timeout_ms)
                return MEGRAY_TIMEOUT;
        }
    }
    return MEGRAY_OK;
}

Status HostCommunicator::_send(const void* sendbuff, size_t size, uint32_t rank,
                               std::shared_ptr<Context> ctx) {
    MEGRAY_CHECK(check_ready(ctx));
    m_stats.calls++;
    m_stats.bytes += size;
    P2POp op{true, rank, const_cast<char*>(static_cast<const char*>(sendbuff)), size, 0, nullptr,
             ctx, nullptr};
#ifdef MEGRAY_WITH_CUDA
    if (ctx->type() == MEGRAY_CTX_CUDA) {
        cudaStream_t stream = static_cast<CudaContext*>(ctx.get())->get_stream();
        op.staging = std::make_shared<std::vector<char>>(size);
        op.host = op.staging->data();
        CUDA_CHECK(cudaMemcpyAsync(op.host, sendbuff, size, cudaMemcpyDeviceToHost, stream));
        CUDA_CHECK(cudaStreamSynchronize(stream));
    }
#endif
    m_queued.push_back(op);
    if (m_grouping)
        return MEGRAY_OK;
    return group_end();
}

Status HostCommunicator::_recv(void* recvbuf, size_t size, uint32_t rank,
                               std::shared_ptr<Context> ctx) {
    MEGRAY_CHECK(check_ready(ctx));
    m_stats.calls++;
    m_stats.bytes += size;
    P2POp op{false, rank, static_cast<char*>(recvbuf), size, 0, nullptr, ctx, nullptr};
#ifdef MEGRAY_WITH_CUDA
    if (ctx->type() == MEGRAY_CTX_CUDA) {
        op.staging = std::make_shared<std::vector<char>>(size);
        op.host = op.staging->data();
        op.device = recvbuf;
    }
#endif
    m_queued.push_back(op);
    if (m_grouping)
        return MEGRAY_OK;
    return group_end();
}

Status HostCommunicator::group_start() {
    if (m_grouping)
        return MEGRAY_INVALID_USAGE;
    m_grouping = true;
    return MEGRAY_OK;
}

Status HostCommunicator::group_end() {
    drain_async();  // stream-ordered jobs use the same barrier state and mailboxes
    m_grouping = false;
    std::vector<P2POp> ops;
    ops.swap(m_queued);
    if (ops.empty())
        return MEGRAY_OK;
    Status s = progress(ops);
    if (s != MEGRAY_OK)
        return fail(s);
#ifdef MEGRAY_WITH_CUDA
    for (P2POp& op : ops) {
        if (op.device != nullptr) {
            cudaStream_t stream = static_cast<CudaContext*>(op.ctx.get())->get_stream();
            CUDA_CHECK(cudaMemcpyAsync(op.device, op.host, op.bytes, cudaMemcpyHostToDevice, stream));
            CUDA_CHECK(cudaStreamSynchronize(stream));
        }
    }
#endif
    return MEGRAY_OK;
}

}  // namespace MegRay
