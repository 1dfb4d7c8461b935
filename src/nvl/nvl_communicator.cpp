#include "nvl/nvl_communicator.h"
#include "nvl/ipc_cache.h"

#include <dlfcn.h>
#include <string.h>
#include <unistd.h>

#include <stdio.h>

#include <algorithm>
#include <random>
#include <string>

#include "megray/cuda_context.h"
#include "megray/options.h"
#include "megray/trace.h"

#ifdef MEGRAY_WITH_NCCL
#include "nccl/nccl_communicator.h"
#endif

namespace MegRay {

using mgk::coll::CommonArgs;
using mgk::coll::DirectArgs;
using mgk::coll::ExchangeArgs;
using mgk::coll::kMaxCtas;
using mgk::coll::kMaxRanks;
using mgk::coll::ReduceArgs;

namespace {

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
size_t round_down(size_t v, size_t a) { return v / a * a; }

int64_t env_i64(const char* name, int64_t dflt) {
    const char* e = getenv(name);
    if (e == nullptr || *e == 0)
        return dflt;
    return atoll(e);
}

// Reads an integer value of `"key": value` from a small JSON text (the tune table written by
// bench/tune.py); returns dflt when the key is absent.
int64_t json_i64(const std::string& text, const char* key, int64_t dflt) {
    const std::string k = std::string("\"") + key + "\"";
    size_t at = text.find(k);
    if (at == std::string::npos)
        return dflt;
    at = text.find(':', at + k.size());
    if (at == std::string::npos)
        return dflt;
    char* end = nullptr;
    const long long v = strtoll(text.c_str() + at + 1, &end, 10);
    return end == text.c_str() + at + 1 ? dflt : static_cast<int64_t>(v);
}

std::string read_file(const std::string& path) {
    std::string out;
    FILE* f = fopen(path.c_str(), "r");
    if (f == nullptr)
        return out;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0)
        out.append(buf, n);
    fclose(f);
    return out;
}

bool is_float(DType t) {
    return t == MEGRAY_FLOAT16 || t == MEGRAY_BFLOAT16 || t == MEGRAY_FLOAT32 ||
           t == MEGRAY_FLOAT64;
}

}  // namespace

NvlInterface* as_nvl(Communicator* comm) { return dynamic_cast<NvlInterface*>(comm); }

NvlCommunicator::NvlCommunicator(uint32_t nranks, uint32_t rank) : Communicator(nranks, rank) {
    const Options& o = global_options();
    m_timeout_ns = static_cast<uint64_t>(o.device_timeout_ms) * 1000000ull;
    m_max_ctas = o.max_ctas > 0 ? std::min(o.max_ctas, kMaxCtas)
                                : static_cast<int>(std::min<int64_t>(kMaxCtas, std::max<int64_t>(1, env_i64("MEGRAY_MAX_CTAS", 64))));
    m_oneshot_bytes = static_cast<size_t>(env_i64("MEGRAY_ONESHOT_BYTES", 256 * 1024));
    m_direct = env_i64("MEGRAY_DIRECT", 1) != 0;
    m_push_exchange = env_i64("MEGRAY_PUSH_EXCHANGE", 1) != 0;
    m_cta_bytes = static_cast<size_t>(env_i64("MEGRAY_CTA_BYTES", 128 * 1024));
    // Measured crossover points (bench/tune.py) override the built-in defaults; explicit
    // environment settings override the table.  The table is the file MEGRAY_TUNE_FILE names, or
    // tune/tune_b200_n<ranks>.json beside the library's directory when that file exists.
    std::string tune_path = o.tune_file;
    if (tune_path.empty() && env_i64("MEGRAY_TUNE_DEFAULT", 1) != 0) {
        Dl_info info;
        if (dladdr(reinterpret_cast<const void*>(&as_nvl), &info) != 0 && info.dli_fname != nullptr) {
            std::string dir(info.dli_fname);
            const size_t slash = dir.rfind('/');
            dir = slash == std::string::npos ? std::string(".") : dir.substr(0, slash);
            tune_path = dir + "/../tune/tune_b200_n" + std::to_string(nranks) + ".json";
        }
    }
    const std::string tune_text = tune_path.empty() ? std::string() : read_file(tune_path);
    if (tune_text.empty()) {
        if (!o.tune_file.empty())
            MEGRAY_WARN("tune file %s is missing or empty", o.tune_file.c_str());
    } else {
        MEGRAY_INFO("NVL backend: thresholds from %s", tune_path.c_str());
        const std::string& t = tune_text;
        if (getenv("MEGRAY_ONESHOT_BYTES") == nullptr)
            m_oneshot_bytes = static_cast<size_t>(json_i64(t, "oneshot_bytes", static_cast<int64_t>(m_oneshot_bytes)));
        if (o.max_ctas <= 0 && getenv("MEGRAY_MAX_CTAS") == nullptr)
            m_max_ctas = std::min<int>(kMaxCtas, static_cast<int>(json_i64(t, "max_ctas", m_max_ctas)));
        if (getenv("MEGRAY_CTA_BYTES") == nullptr)
            m_cta_bytes = static_cast<size_t>(json_i64(t, "cta_bytes", static_cast<int64_t>(m_cta_bytes)));
        m_nvls_min_bytes = static_cast<size_t>(json_i64(t, "nvls_min_bytes", 0));
    }
    if (m_cta_bytes < 1024)
        m_cta_bytes = 1024;
    int64_t bcast_chunk_tuned = -1;
    // small-message limits (payload bytes per source / destination pair), per operation
    static const char* const kKindNames[8] = {"all_reduce", "reduce_scatter", "all_gather", "all_to_all",
                                              "broadcast",  "reduce",         "gather",     "scatter"};
    static const size_t kLLDefaults[8] = {65536, 65536, 65536, 65536, 65536, 65536, 65536, 65536};
    const int64_t ll_all = env_i64("MEGRAY_LL_BYTES", -1);
    for (int k = 0; k < 8; ++k) {
        int64_t v = static_cast<int64_t>(kLLDefaults[k]);
        if (!tune_text.empty())
            v = json_i64(tune_text, (std::string("ll_") + kKindNames[k]).c_str(), v);
        if (ll_all >= 0)
            v = ll_all;
        m_ll_bytes[k] = std::min<size_t>(static_cast<size_t>(std::max<int64_t>(v, 0)), mgk::coll::kLLMaxBytes);
    }
    m_direct_cta_bytes = static_cast<size_t>(env_i64("MEGRAY_DIRECT_CTA_BYTES", 32 * 1024));
    if (!tune_text.empty() && getenv("MEGRAY_DIRECT_CTA_BYTES") == nullptr)
        m_direct_cta_bytes = static_cast<size_t>(json_i64(tune_text, "direct_cta_bytes", static_cast<int64_t>(m_direct_cta_bytes)));
    if (m_direct_cta_bytes < 4096)
        m_direct_cta_bytes = 4096;
    if (!tune_text.empty() && getenv("MEGRAY_BCAST_CHUNK") == nullptr)
        bcast_chunk_tuned = json_i64(tune_text, "bcast_chunk_bytes", -1);
    m_phases = env_i64("MEGRAY_PHASES", 0) != 0;
    m_spin_sleep_ns = static_cast<uint32_t>(env_i64("MEGRAY_SPIN_SLEEP_NS", 0));
    m_bcast_pull = env_i64("MEGRAY_BCAST_PULL", 0) != 0;
    if (!tune_text.empty() && getenv("MEGRAY_BCAST_PULL") == nullptr)
        m_bcast_pull = json_i64(tune_text, "bcast_pull", m_bcast_pull ? 1 : 0) != 0;
    m_bcast_pull_min = static_cast<size_t>(env_i64("MEGRAY_BCAST_PULL_MIN", 0));
    if (!tune_text.empty() && getenv("MEGRAY_BCAST_PULL_MIN") == nullptr)
        m_bcast_pull_min = static_cast<size_t>(json_i64(tune_text, "bcast_pull_min_bytes", static_cast<int64_t>(m_bcast_pull_min)));
    m_reduce_mode = static_cast<int>(env_i64("MEGRAY_REDUCE_MODE", 0));
    if (!tune_text.empty() && getenv("MEGRAY_REDUCE_MODE") == nullptr)
        m_reduce_mode = static_cast<int>(json_i64(tune_text, "reduce_mode", m_reduce_mode));
    m_reduce_staged_min = static_cast<size_t>(env_i64("MEGRAY_REDUCE_STAGED_MIN", 8 << 20));
    if (!tune_text.empty() && getenv("MEGRAY_REDUCE_STAGED_MIN") == nullptr)
        m_reduce_staged_min = static_cast<size_t>(json_i64(tune_text, "reduce_staged_min_bytes", static_cast<int64_t>(m_reduce_staged_min)));
    if (!tune_text.empty() && getenv("MEGRAY_SPIN_SLEEP_NS") == nullptr)
        m_spin_sleep_ns = static_cast<uint32_t>(json_i64(tune_text, "spin_sleep_ns", m_spin_sleep_ns));
    m_guard_shrink = env_i64("MEGRAY_DEBUG_BOUNDS_SELFTEST", 0) != 0;
    m_bcast_chunk = static_cast<uint32_t>(round_up(
            static_cast<size_t>(bcast_chunk_tuned > 0 ? bcast_chunk_tuned : env_i64("MEGRAY_BCAST_CHUNK", 64 * 1024)), 16));
    if (m_bcast_chunk < 4096)
        m_bcast_chunk = 4096;
    if (o.algo == "oneshot")
        m_oneshot_bytes = ~static_cast<size_t>(0);
    else if (o.algo == "twoshot")
        m_oneshot_bytes = 0;
}

NvlCommunicator::~NvlCommunicator() {
    if (m_ready) {
        cudaSetDevice(m_heap.device());
        cudaDeviceSynchronize();
    }
    m_p2p.reset();
    m_p2p_ctx.reset();
    if (m_p2p_stream != nullptr) {
        cudaStreamDestroy(m_p2p_stream);
        cudaEventDestroy(m_p2p_fork);
        cudaEventDestroy(m_p2p_done);
    }
    for (void*& b : m_bounce) {
        if (b != nullptr)
            cudaFree(b);
        b = nullptr;
    }
    if (m_last_event != nullptr)
        cudaEventDestroy(m_last_event);
    if (m_status_host != nullptr)
        cudaFreeHost(m_status_host);
    // peers may still be inside their last kernel reading this rank's heap: meet first
    if (m_ready && m_client && m_client->connected() && !m_aborted.load())
        m_client->barrier();
    m_ipc.reset();  // stops the helper thread and closes the mappings of the peers' allocations
    for (Registration& r : m_regs)
        drop_registration(r);
    m_regs.clear();
    m_heap.destroy();
}

Status NvlCommunicator::check_cuda(cudaError_t e) {
    if (e == cudaSuccess)
        return MEGRAY_OK;
    MEGRAY_ERROR("cuda error [%d]: %s", e, cudaGetErrorString(e));
    if (m_error == MEGRAY_OK)
        m_error = MEGRAY_CUDA_ERR;
    return MEGRAY_CUDA_ERR;
}

Status NvlCommunicator::do_init(BcastCallback cb) {
    // No server was given: rank 0 starts a private one and publishes its address
    // through the caller's broadcast.
    struct {
        char ip[64];
        int32_t port;
    } where;
    memset(&where, 0, sizeof(where));
    if (m_rank == 0) {
        m_own_server.reset(new Server(m_nranks, 0));
        char* ip = get_host_ip();
        snprintf(where.ip, sizeof(where.ip), "%s", ip != nullptr ? ip : "127.0.0.1");
        delete[] ip;
        where.port = m_own_server->port();
    }
    cb(reinterpret_cast<char*>(&where), sizeof(where));
    where.ip[sizeof(where.ip) - 1] = 0;
    m_client = std::make_shared<Client>(m_nranks, m_rank);
    Status s = m_client->connect(where.ip, where.port);
    if (s != MEGRAY_OK && strcmp(where.ip, "127.0.0.1") != 0)
        s = m_client->connect("127.0.0.1", where.port);
    MEGRAY_CHECK(s);
    return do_init();
}

Status NvlCommunicator::do_init() {
    if (m_nranks > static_cast<uint32_t>(kMaxRanks)) {
        MEGRAY_ERROR("NVL backend supports up to %d ranks", kMaxRanks);
        return MEGRAY_INVALID_ARGUMENT;
    }
    const Options& o = global_options();
    // a name for this group on this machine
    uint64_t gid = 0;
    if (m_rank == 0) {
        std::random_device rd;
        gid = (static_cast<uint64_t>(rd()) << 32) ^ rd() ^ (static_cast<uint64_t>(getpid()) << 20);
    }
    MEGRAY_CHECK(m_client->broadcast(&gid, &gid, sizeof(gid), 0));
    char group[32];
    snprintf(group, sizeof(group), "%016llx", static_cast<unsigned long long>(gid));

    const size_t heap_bytes = static_cast<size_t>(o.heap_mb) << 20;
    MEGRAY_CHECK(m_heap.create(m_client.get(), m_nranks, m_rank, heap_bytes, group, o.nvls));

    m_ws_bytes = static_cast<size_t>(env_i64("MEGRAY_WORKSPACE_MB", 0)) << 20;
    if (m_ws_bytes == 0)
        m_ws_bytes = std::min<size_t>(192ull << 20, m_heap.bytes() / 8);
    m_ws_bytes = round_down(m_ws_bytes, 4096);
    // canary zones before, between and after the two workspaces
    m_user_off = round_up(kWorkspaceOff + 3 * kCanaryBytes + 2 * m_ws_bytes, 1 << 20);
    if (m_user_off >= m_heap.bytes()) {
        MEGRAY_ERROR("heap of %zu bytes is too small for two %zu-byte workspaces", m_heap.bytes(),
                     m_ws_bytes);
        return MEGRAY_INVALID_ARGUMENT;
    }
    m_user_top = m_user_off;

    for (int z = 0; z < 3; ++z)
        CUDA_CHECK(cudaMemset(m_heap.local() + canary_off(z), kCanaryByte, kCanaryBytes));
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaHostAlloc(reinterpret_cast<void**>(&m_status_host), 64, cudaHostAllocMapped));
    memset(m_status_host, 0, 64);
    CUDA_CHECK(cudaHostGetDevicePointer(reinterpret_cast<void**>(&m_status_dev), m_status_host, 0));
    CUDA_CHECK(cudaEventCreateWithFlags(&m_last_event, cudaEventDisableTiming));

    // Ranks that are threads of one process address each other's device memory directly once peer
    // access is on: then ordinary cudaMalloc buffers need neither staging nor registration.
    {
        int32_t mine = m_heap.same_process() && env_i64("MEGRAY_EXCHANGE", 1) != 0 ? 1 : 0;
        for (uint32_t q = 0; q < m_nranks && mine; ++q) {
            if (q == m_rank)
                continue;
            cudaError_t e = cudaDeviceEnablePeerAccess(m_heap.peer_device(q), 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                mine = 0;
            (void)cudaGetLastError();
        }
        if (drv::api() == nullptr)
            mine = 0;
        std::vector<int32_t> all(m_nranks, 0);
        MEGRAY_CHECK(m_client->allgather(&mine, all.data(), sizeof(int32_t)));
        m_xchg = true;
        for (uint32_t q = 0; q < m_nranks; ++q)
            m_xchg = m_xchg && all[q] != 0;
    }
    // Ranks in separate processes: allocations are exported and mapped on first use, after which
    // the same kernels run on them (MEGRAY_IPC_CACHE=0 keeps ordinary buffers on the staged paths).
    if (!m_xchg && m_nranks > 1 && env_i64("MEGRAY_IPC_CACHE", 1) != 0 && env_i64("MEGRAY_EXCHANGE", 1) != 0) {
        static_assert(IpcCache::kMaxExports == mgk::coll::kImportEntries, "table geometry");
        static_assert(IpcCache::kEntryNull == mgk::coll::kWordEntryNull && IpcCache::kEntryHeap == mgk::coll::kWordEntryHeap,
                      "word encoding");
        m_ipc.reset(new IpcCache());
        if (m_ipc->init(*m_client, m_nranks, m_rank, m_heap.device())) {
            m_xchg = true;
        } else {
            m_ipc.reset();
            MEGRAY_INFO("NVL backend: no shared export logs; ordinary buffers take the staged paths");
        }
    }

#ifdef MEGRAY_WITH_NCCL
    // point-to-point engine
    if (m_nranks > 1 && env_i64("MEGRAY_NVL_P2P", 1) != 0) {
        m_p2p.reset(new NcclCommunicator(m_nranks, m_rank));
        std::shared_ptr<Client> client = m_client;
        Status s = m_p2p->init([client](char* buf, size_t len) { client->broadcast(buf, buf, len, 0); });
        if (s != MEGRAY_OK) {
            MEGRAY_WARN("NCCL point-to-point engine unavailable (status %d): send/recv disabled", s);
            m_p2p.reset();
        }
    }
#endif
    m_ready = true;
    return m_client->barrier();
}

Status NvlCommunicator::begin(const std::shared_ptr<Context>& ctx, cudaStream_t* stream) {
    if (!ctx || ctx->type() != MEGRAY_CTX_CUDA) {
        MEGRAY_ERROR("NVL backend needs a CudaContext");
        return MEGRAY_INVALID_ARGUMENT;
    }
    *stream = static_cast<CudaContext*>(ctx.get())->get_stream();
    return begin_on(*stream);
}

Status NvlCommunicator::begin_on(cudaStream_t s) {
    cudaStream_t* stream = &s;
    if (!m_ready) {
        MEGRAY_ERROR("communicator used before init");
        return MEGRAY_INVALID_USAGE;
    }
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    if (*m_status_host != 0) {  // an earlier kernel gave up waiting
        adopt_device_status();
        return m_error;
    }
    if (m_error != MEGRAY_OK)
        return m_error;
    // Launches of one communicator share staging memory and flag epochs: they must
    // run in issue order even when the caller switches streams.
    if (m_has_last && m_last_stream != *stream) {
        CUDA_CHECK(cudaEventRecord(m_last_event, m_last_stream));
        CUDA_CHECK(cudaStreamWaitEvent(*stream, m_last_event, 0));
    }
    m_stats.calls++;
    return MEGRAY_OK;
}

// A kernel reported a failure: make it the communicator's error, once.  For a refused access
// (bounds-checked build) say which one it was.
void NvlCommunicator::adopt_device_status() {
    if (m_error != MEGRAY_OK)
        return;
    m_error = static_cast<Status>(*m_status_host);
    m_stats.timeouts++;
    if (m_error == MEGRAY_OUT_OF_BOUNDS) {
        uint64_t rec[3] = {0, 0, 0};
        (void)cudaDeviceSynchronize();  // (the record is written right after the status)
        if (cudaMemcpy(rec, m_heap.local() + mgk::coll::kDebugOff, sizeof(rec), cudaMemcpyDeviceToHost) == cudaSuccess)
            MEGRAY_ERROR("rank %u: the range guard refused an access of %llu bytes at %p (collectives.cu line %u); "
                         "declared buffers: in %p + %zu, out %p + %zu, peers' in %zu, out %zu",
                         m_rank, static_cast<unsigned long long>(rec[1]), reinterpret_cast<void*>(rec[0]),
                         static_cast<unsigned>(rec[2] & 0xffffffffu), m_guard.in, m_guard.in_bytes, m_guard.out,
                         m_guard.out_bytes, m_guard.peer_in_bytes, m_guard.peer_out_bytes);
        (void)cudaGetLastError();
    } else {
        uint64_t rec[3] = {0, 0, 0};
        (void)cudaDeviceSynchronize();
        if (cudaMemcpy(rec, m_heap.local() + mgk::coll::kDebugOff + 32, sizeof(rec), cudaMemcpyDeviceToHost) == cudaSuccess &&
            rec[0] != 0)
            MEGRAY_ERROR("rank %u: a collective kernel gave up with status %d at collectives.cu line %u (what %u, detail 0x%x)",
                         m_rank, static_cast<int>(m_error), static_cast<unsigned>(rec[0]), static_cast<unsigned>(rec[1] >> 32),
                         static_cast<unsigned>(rec[1] & 0xffffffffu));
        else
            MEGRAY_ERROR("rank %u: a kernel reported status %d", m_rank, static_cast<int>(m_error));
        (void)cudaGetLastError();
    }
}

void NvlCommunicator::after_launch(cudaStream_t stream) {
    m_stats.kernels++;
    m_last_stream = stream;
    m_has_last = true;
}

CommonArgs NvlCommunicator::common_args(uint32_t epochs) {
    CommonArgs c;
    memset(&c, 0, sizeof(c));
    for (uint32_t q = 0; q < m_nranks; ++q)
        c.peers.heap[q] = m_heap.base(q);
    c.nranks = static_cast<int>(m_nranks);
    c.rank = static_cast<int>(m_rank);
    c.epoch = m_epoch;
    m_epoch += epochs;  // a launch uses at most two barriers
    c.timeout_ns = m_timeout_ns;
    c.status = m_status_dev;
    c.flag_off = kFlagOff;
    c.heap_bytes = m_heap.bytes();
    c.phases = m_phases ? 1 : 0;
    c.spin_sleep_ns = m_spin_sleep_ns;
    c.guard_in = m_guard.in;
    c.guard_in_bytes = m_guard.in_bytes;
    c.guard_out = m_guard.out;
    c.guard_out_bytes = m_guard.out_bytes;
    c.guard_peer_in_bytes = m_guard.peer_in_bytes;
    c.guard_peer_out_bytes = m_guard.peer_out_bytes;
    return c;
}

Status NvlCommunicator::fused_begin(void* stream) { return begin_on(static_cast<cudaStream_t>(stream)); }

void NvlCommunicator::fused_end(void* stream) { after_launch(static_cast<cudaStream_t>(stream)); }

void NvlCommunicator::set_guard(const void* in, size_t in_bytes, void* out, size_t out_bytes) {
    m_guard.in = in;
    m_guard.in_bytes = in != nullptr ? in_bytes : 0;
    m_guard.out = out;
    m_guard.out_bytes = out != nullptr ? out_bytes : 0;
    m_guard.peer_in_bytes = in_bytes;
    m_guard.peer_out_bytes = out_bytes;
    if (m_guard_shrink) {
        // self-test of the bounds-checked build: claim that the buffers are half as long as they
        // are, so that the guard must refuse (and skip) accesses that are in fact harmless
        m_guard.in_bytes /= 2;
        m_guard.out_bytes /= 2;
        m_guard.peer_in_bytes /= 2;
        m_guard.peer_out_bytes /= 2;
    }
}

uint32_t NvlCommunicator::fused_call_count(const void* flags) {
    if (!in_heap(flags, 1))
        return 0;
    const size_t off = static_cast<size_t>(static_cast<const char*>(flags) - m_heap.local());
    return ++m_fused_calls[off];
}

uint32_t NvlCommunicator::reserve_epochs(uint32_t count) {
    const uint32_t e = m_epoch;
    m_epoch += count;
    return e;
}

size_t NvlCommunicator::canary_off(int zone) const {
    return kWorkspaceOff + static_cast<size_t>(zone) * (kCanaryBytes + m_ws_bytes);
}

Status NvlCommunicator::check_canaries() {
    if (!m_ready)
        return MEGRAY_INVALID_USAGE;
    CUDA_CHECK(cudaDeviceSynchronize());
    std::vector<unsigned char> host(kCanaryBytes);
    for (int z = 0; z < 3; ++z) {
        CUDA_CHECK(cudaMemcpy(host.data(), m_heap.local() + canary_off(z), kCanaryBytes, cudaMemcpyDeviceToHost));
        for (size_t i = 0; i < kCanaryBytes; ++i) {
            if (host[i] != kCanaryByte) {
                MEGRAY_ERROR("rank %u: canary zone %d around the staging workspaces was overwritten at byte %zu", m_rank,
                             z, i);
                if (m_error == MEGRAY_OK)
                    m_error = MEGRAY_OUT_OF_BOUNDS;
                return MEGRAY_OUT_OF_BOUNDS;
            }
        }
    }
    return MEGRAY_OK;
}

int NvlCommunicator::read_phase_stamps(uint64_t* out, int max) {
    if (!m_ready || !m_phases || out == nullptr)
        return 0;
    cudaDeviceSynchronize();
    uint64_t all[mgk::coll::kMaxPhases] = {};
    if (cudaMemcpy(all, m_heap.local() + mgk::coll::kPhaseOff, sizeof(all), cudaMemcpyDeviceToHost) != cudaSuccess)
        return 0;
    // stamps of one kernel increase; a smaller value belongs to an earlier kernel with more phases
    int n = 0;
    while (n < mgk::coll::kMaxPhases && n < max && all[n] != 0 && (n == 0 || all[n] >= all[n - 1])) {
        out[n] = all[n];
        ++n;
    }
    return n;
}

size_t NvlCommunicator::workspace_off() {
    const size_t off = kWorkspaceOff + kCanaryBytes + static_cast<size_t>(m_parity) * (m_ws_bytes + kCanaryBytes);
    m_parity ^= 1;
    return off;
}

int NvlCommunicator::pick_ctas(size_t bytes) const {
    // enough CTAs to keep the links busy, few enough that flag traffic stays small
    size_t want = (bytes + m_cta_bytes - 1) / m_cta_bytes;
    if (want < 1)
        want = 1;
    return static_cast<int>(std::min<size_t>(want, static_cast<size_t>(m_max_ctas)));
}


// ------------------------------------------------------------------ direct (zero-copy) paths

// True if every peer's kernels can address [p, p + bytes): it lies in the symmetric heap or in a
// registered buffer (and is 16-byte aligned).
bool NvlCommunicator::aligned_heap(const void* p, size_t bytes) {
    char* base[mgk::coll::kMaxRanks];
    size_t off;
    return peer_view(p, bytes, base, &off);
}

Status NvlCommunicator::direct_launch(int kind, const void* in, void* out, size_t len, DType in_dtype,
                                      DType out_dtype, float scale, ReduceOp op, cudaStream_t stream) {
    DirectArgs a;
    memset(&a, 0, sizeof(a));
    a.c = common_args();
    a.kind = kind;
    a.len = len;
    a.scale = scale;
    a.in_dtype = in_dtype;
    a.out_dtype = out_dtype;
    a.op = op;
    size_t bytes = len * get_dtype_size(in_dtype);
    size_t in_off = SIZE_MAX, out_off = SIZE_MAX;
    char* in_base[mgk::coll::kMaxRanks] = {};
    bool ok = true;
    if (kind == mgk::coll::DIRECT_ALL_GATHER || kind == mgk::coll::DIRECT_ALL_TO_ALL) {
        a.in_local = in;
        bytes *= m_nranks;
        ok = peer_view(out, bytes, a.out_base, &out_off);
        in_off = 0;  // (no multimem load on these paths)
    } else {
        const size_t in_bytes = kind == mgk::coll::DIRECT_ALL_REDUCE ? bytes : bytes * m_nranks;
        ok = peer_view(in, in_bytes, in_base, &in_off);
        for (uint32_t q = 0; q < m_nranks; ++q)
            a.in_base[q] = in_base[q];
        if (kind == mgk::coll::DIRECT_ALL_REDUCE) {
            ok = ok && peer_view(out, len * get_dtype_size(out_dtype), a.out_base, &out_off);
        } else {
            a.out_local = out;
            out_off = 0;
            bytes *= m_nranks;
        }
    }
    if (!ok)
        return MEGRAY_INVALID_ARGUMENT;
    // the NVSwitch paths need both buffers inside the multicast-mapped heap
    const bool nvls = m_heap.multicast() != nullptr && in_off != SIZE_MAX && out_off != SIZE_MAX &&
                      bytes >= m_nvls_min_bytes && kind != mgk::coll::DIRECT_ALL_TO_ALL &&
                      (kind == mgk::coll::DIRECT_ALL_GATHER || mgk::coll::nvls_supports(in_dtype, out_dtype, op));
    a.mc_base = nvls ? m_heap.multicast() : nullptr;
    a.heap_bytes = m_heap.bytes();
    // single-pass kernels are latency-bound per CTA: smaller shares, more CTAs
    const int ctas = static_cast<int>(std::min<size_t>(std::max<size_t>(1, bytes / m_direct_cta_bytes),
                                                       static_cast<size_t>(2 * m_max_ctas > kMaxCtas ? kMaxCtas : 2 * m_max_ctas)));
    MEGRAY_CHECK(check_cuda(mgk::coll::launch_direct(a, ctas, 512, stream)));
    after_launch(stream);
    if (nvls)
        m_stats.algo_nvls++;
    else
        m_stats.algo_twoshot++;
    return MEGRAY_OK;
}


// ------------------------------------------------------------------ small messages (flagged words)

void NvlCommunicator::ll_ticket(uint32_t* seq, size_t* slot_off, size_t* slot_stride) {
    if (++m_ll_seq == 0)
        m_ll_seq = 1;
    *seq = m_ll_seq;
    *slot_off = kLLOff + static_cast<size_t>(m_ll_parity) * kMaxRanks * mgk::coll::kLLSlotBytes;
    *slot_stride = mgk::coll::kLLSlotBytes;
    m_ll_parity ^= 1;
}

Status NvlCommunicator::ll_launch(mgk::coll::LLArgs& a, cudaStream_t stream) {
    a.c = common_args(0);  // no barrier: no epochs
    const int parity = m_ll_parity;
    size_t slot_off = 0, slot_stride = 0;
    ll_ticket(&a.seq, &slot_off, &slot_stride);
    a.slot_off = slot_off;
    a.token_off = mgk::coll::kTokenOff + static_cast<size_t>(parity) * kMaxRanks * 8;
    const size_t units = (a.bytes + 15) / 16;
    const size_t fan = std::max<size_t>(
            1, std::max<size_t>(__builtin_popcount(a.send_mask), __builtin_popcount(a.recv_mask) + (a.self ? 1 : 0)));
    const size_t work = units * fan;
    // latency-bound at the small end (one small CTA), store-bandwidth-bound at the large end
    const int threads = work <= 128 ? 128 : 256;
    const int ctas = static_cast<int>(std::min<size_t>(64, std::max<size_t>(1, (work + 1023) / 1024)));
    MEGRAY_CHECK(check_cuda(mgk::coll::launch_ll(a, ctas, threads, stream)));
    after_launch(stream);
    m_stats.algo_ll++;
    return MEGRAY_OK;
}

// ------------------------------------------------------------------ single pass on the call's own buffers

bool NvlCommunicator::peer_addressable(const void* p, size_t bytes) {
    if (p == nullptr || bytes == 0)
        return true;
    if (in_heap(p, bytes))
        return true;
    const drv::Api* api = drv::api();
    if (api == nullptr)
        return false;
    // cudaMalloc memory of this rank's device: peers that enabled peer access to the device reach it
    unsigned int mem_type = 0;
    int ordinal = -1;
    int legacy = 0;
    CUdeviceptr start = 0;
    size_t size = 0;
    CUpointer_attribute attrs[5] = {CU_POINTER_ATTRIBUTE_MEMORY_TYPE, CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL,
                                    CU_POINTER_ATTRIBUTE_IS_LEGACY_CUDA_IPC_CAPABLE,
                                    CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, CU_POINTER_ATTRIBUTE_RANGE_SIZE};
    void* vals[5] = {&mem_type, &ordinal, &legacy, &start, &size};
    if (api->PointerGetAttributes(5, attrs, vals, reinterpret_cast<CUdeviceptr>(p)) != CUDA_SUCCESS)
        return false;
    const CUdeviceptr at = reinterpret_cast<CUdeviceptr>(p);
    return mem_type == CU_MEMORYTYPE_DEVICE && ordinal == m_heap.device() && legacy != 0 && at >= start &&
           at + bytes <= start + size;
}

void* NvlCommunicator::bounce(int which, size_t bytes) {
    if (m_ipc != nullptr)  // separate processes: the buffers every peer mapped at init
        return bytes <= m_ipc->bounce_bytes() ? m_ipc->bounce(which) : nullptr;
    if (m_bounce_cap[which] >= bytes)
        return m_bounce[which];
    // rare: a buffer the peers cannot address (pool or virtual-memory allocations, host memory)
    cudaDeviceSynchronize();
    if (m_bounce[which] != nullptr)
        cudaFree(m_bounce[which]);
    m_bounce[which] = nullptr;
    m_bounce_cap[which] = 0;
    const size_t cap = round_up(bytes, 2u << 20);
    if (cudaMalloc(&m_bounce[which], cap) != cudaSuccess) {
        (void)cudaGetLastError();
        m_bounce[which] = nullptr;
        return nullptr;
    }
    m_bounce_cap[which] = cap;
    return m_bounce[which];
}

// Ranks in separate processes: may this call take the single-pass kernels?  Up to
// auto_max_bytes() per buffer always (allocations are exported on first use, a large one is
// replaced by a bounce buffer).  Above, only when every buffer this rank passes lies in the heap
// or in an allocation that every peer has mapped already (register_buffer sees to that):
// mapping a large allocation can wait for the importing device, and a kernel that waits for the
// mapping would then wait for itself.  The rule depends on sizes and on what the program did on
// every rank alike, so all ranks take the same path.
bool NvlCommunicator::exchange_fits(const void* in, size_t in_bytes, const void* out, size_t out_bytes) {
    if (m_ipc == nullptr)
        return true;
    if (std::max(in != nullptr ? in_bytes : 0, out != nullptr ? out_bytes : 0) <= m_ipc->auto_max_bytes())
        return true;
    auto fine = [&](const void* p, size_t bytes) {
        return p == nullptr || in_heap(p, bytes) || m_ipc->mapped_everywhere(p, bytes);
    };
    return fine(in, in_bytes) && fine(out, out_bytes);
}

Status NvlCommunicator::exchange_launch(int kind, const void* in, size_t in_bytes, bool in_shared, void* out,
                                        size_t out_bytes, bool out_shared, size_t len, DType in_dtype,
                                        DType out_dtype, float scale, ReduceOp op, uint32_t root,
                                        cudaStream_t stream) {
    const void* in_use = in;
    void* out_use = out;
    bool copy_back = false;
    // what this rank tells its peers about the two buffers: the address (ranks of one process),
    // or the allocation's export entry and the offset inside it (ranks in separate processes)
    uint64_t in_word = 0, out_word = 0;
    auto describe = [&](const void* p, size_t bytes, uint64_t* word) {
        if (m_ipc == nullptr) {
            *word = reinterpret_cast<uint64_t>(p);
            return peer_addressable(p, bytes);
        }
        if (p == nullptr) {
            *word = IpcCache::encode(IpcCache::kEntryNull, 0);
            return true;
        }
        if (in_heap(p, bytes)) {
            *word = IpcCache::encode(IpcCache::kEntryHeap, static_cast<uint64_t>(static_cast<const char*>(p) - m_heap.local()));
            return true;
        }
        // (an allocation the peers have not all mapped yet is exported now and replaced by a
        // bounce buffer for this call: nothing waits for the mapping)
        return m_ipc->resolve_mapped(p, bytes, word);
    };
    if (in == nullptr || !in_shared) {
        // (peers never touch it: nothing to describe)
        in_word = m_ipc ? IpcCache::encode(IpcCache::kEntryNull, 0) : reinterpret_cast<uint64_t>(in);
    } else if (!describe(in, in_bytes, &in_word)) {
        void* b = bounce(0, in_bytes);
        if (b == nullptr || !describe(b, in_bytes, &in_word))
            return MEGRAY_CUDA_ERR;
        MEGRAY_CHECK(check_cuda(cudaMemcpyAsync(b, in, in_bytes, cudaMemcpyDefault, stream)));
        in_use = b;
    }
    if (out == nullptr || !out_shared) {
        out_word = m_ipc ? IpcCache::encode(IpcCache::kEntryNull, 0) : reinterpret_cast<uint64_t>(out);
    } else if (!describe(out, out_bytes, &out_word)) {
        void* b = bounce(1, out_bytes);
        if (b == nullptr || !describe(b, out_bytes, &out_word))
            return MEGRAY_CUDA_ERR;
        out_use = b;
        copy_back = true;
    }
    set_guard(in_use, in_bytes, out_use, out_bytes);
    DirectArgs a;
    memset(&a, 0, sizeof(a));
    a.c = common_args();
    a.kind = kind;
    a.len = len;
    a.scale = scale;
    a.in_dtype = in_dtype;
    a.out_dtype = out_dtype;
    a.op = op;
    a.root = static_cast<int>(root);
    a.exchange = m_ipc ? 2 : 1;
    a.in_word = in_word;
    a.out_word = out_word;
    a.import_table = m_ipc ? m_ipc->table() : nullptr;
    a.parity = m_xchg_parity;
    m_xchg_parity ^= 1;
    a.in_local = in_use;
    a.out_local = out_use;
    a.heap_bytes = m_heap.bytes();
    const size_t ein = get_dtype_size(in_dtype);
    // bytes that cross this rank's links, for sizing the grid
    size_t work = len * ein;
    const bool reducing = kind == mgk::coll::DIRECT_ALL_REDUCE || kind == mgk::coll::DIRECT_REDUCE_SCATTER ||
                          kind == mgk::coll::DIRECT_REDUCE;
    if (kind == mgk::coll::DIRECT_REDUCE_SCATTER || kind == mgk::coll::DIRECT_ALL_GATHER ||
        kind == mgk::coll::DIRECT_ALL_TO_ALL || kind == mgk::coll::DIRECT_SCATTER)
        work *= m_nranks;
    const bool nvls = m_heap.multicast() != nullptr && work >= m_nvls_min_bytes &&
                      (kind == mgk::coll::DIRECT_ALL_GATHER ||
                       (reducing && mgk::coll::nvls_supports(in_dtype, out_dtype, op)));
    a.mc_base = nvls ? m_heap.multicast() : nullptr;
    const int max_ctas = 2 * m_max_ctas > kMaxCtas ? kMaxCtas : 2 * m_max_ctas;
    int ctas = static_cast<int>(std::min<size_t>(std::max<size_t>(1, work / m_direct_cta_bytes), static_cast<size_t>(max_ctas)));
    if (kind == mgk::coll::DIRECT_BROADCAST) {
        // a CTA moves its share of every slice in chunks; small shares are not worth a CTA
        const size_t slice = m_nranks > 1 ? (work + m_nranks - 2) / (m_nranks - 1) : work;
        ctas = static_cast<int>(std::min<size_t>(std::max<size_t>(1, slice / (m_direct_cta_bytes / 2)), static_cast<size_t>(max_ctas)));
        a.chunk_bytes = m_bcast_chunk;
        a.chunk_base = m_chunk_seq;
        a.bcast_pull = m_bcast_pull && work >= m_bcast_pull_min ? 1 : 0;
        m_chunk_seq += mgk::coll::bcast_plan(work, static_cast<int>(m_nranks), ctas, a.chunk_bytes).chunks;
    }
    if (kind == mgk::coll::DIRECT_REDUCE && m_nranks > 2 && m_reduce_mode != 0 && work >= m_reduce_staged_min && !nvls &&
        get_dtype_size(out_dtype) == ein) {
        // large messages: the root pushes its input into staging slots of the reducing ranks
        const size_t slice = (work + m_nranks - 2) / (m_nranks - 1);
        const int want = static_cast<int>(std::min<size_t>(std::max<size_t>(1, slice / (m_direct_cta_bytes / 2)), static_cast<size_t>(max_ctas)));
        const size_t slots = std::min<size_t>(8, m_ws_bytes / (static_cast<size_t>(want) * m_bcast_chunk));
        if (m_reduce_mode == 3) {
            // in steps: the grid of the plain form; a CTA's share of a slice in `steps` pieces, two
            // slots of one piece per CTA in every reducer's workspace
            const size_t v16 = 16 / ein;
            const size_t se = round_up((len + m_nranks - 2) / (m_nranks - 1), v16);
            const size_t per_cta = round_up((se + ctas - 1) / ctas, v16);
            size_t steps = static_cast<size_t>(std::max<int64_t>(2, env_i64("MEGRAY_REDUCE_STEPS", 8)));
            size_t piece = round_up((per_cta + steps - 1) / steps, v16);
            while (2 * static_cast<size_t>(ctas) * piece * ein > m_ws_bytes && steps < 256) {
                steps *= 2;
                piece = round_up((per_cta + steps - 1) / steps, v16);
            }
            steps = (per_cta + piece - 1) / piece;  // (the last pieces may be empty otherwise)
            if (2 * static_cast<size_t>(ctas) * piece * ein <= m_ws_bytes && steps >= 1) {
                a.chunk_bytes = static_cast<uint32_t>(piece * ein);
                a.stage_off = workspace_off();
                a.stage_slots = static_cast<uint32_t>(steps);
                a.reduce_mode = 3;
                m_epoch += static_cast<uint32_t>(steps);  // one barrier per step, beyond the usual two
            }
        } else if (slots >= 2) {
            ctas = want;
            a.chunk_bytes = m_bcast_chunk;
            a.chunk_base = m_chunk_seq;
            m_chunk_seq += mgk::coll::reduce_plan(len, static_cast<int>(m_nranks), ctas, a.chunk_bytes,
                                                  static_cast<uint32_t>(ein)).chunks;
            a.stage_off = workspace_off();
            a.stage_slots = static_cast<uint32_t>(slots);
            a.reduce_mode = m_reduce_mode;
        }
    }
    MEGRAY_CHECK(check_cuda(mgk::coll::launch_direct(a, ctas, 512, stream)));
    after_launch(stream);
    if (nvls)
        m_stats.algo_nvls++;
    m_stats.algo_direct++;
    if (copy_back)
        MEGRAY_CHECK(check_cuda(cudaMemcpyAsync(out, out_use, out_bytes, cudaMemcpyDefault, stream)));
    return MEGRAY_OK;
}

// ------------------------------------------------------------------ reduce family

Status NvlCommunicator::reduce_impl(ReduceKind kind, const void* in, void* out, size_t len,
                                    DType in_dtype, DType out_dtype, float scale, ReduceOp op,
                                    uint32_t root, cudaStream_t stream) {
    const size_t ein = get_dtype_size(in_dtype), eout = get_dtype_size(out_dtype);
    const uint32_t n = m_nranks;
    m_stats.bytes += len * ein;
    if (len == 0)
        return MEGRAY_OK;
    const bool wants_out = kind != ReduceKind::Reduce || m_rank == root;
    if (in == nullptr || (wants_out && out == nullptr))
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(in, len * ein * (kind == ReduceKind::ReduceScatter ? n : 1), wants_out ? out : nullptr, len * eout);

    // Largest slice (elements) whose n staging slots plus reduced slice fit one workspace.
    const size_t se_max = round_down((m_ws_bytes - 16 * (n + 1)) / (n * ein + eout), 16);
    if (se_max == 0)
        return MEGRAY_INVALID_ARGUMENT;

    ReduceArgs a;
    memset(&a, 0, sizeof(a));
    a.scale = scale;
    a.in_dtype = in_dtype;
    a.out_dtype = out_dtype;
    a.op = op;
    a.do_gather = wants_out ? 1 : 0;

    const char* inb = static_cast<const char*>(in);
    char* outb = static_cast<char*>(out);

    // Small messages travel as flagged words: one launch, no barrier.
    {
        const int k = kind == ReduceKind::AllReduce ? mgk::coll::DIRECT_ALL_REDUCE
                      : kind == ReduceKind::Reduce  ? mgk::coll::DIRECT_REDUCE
                                                    : mgk::coll::DIRECT_REDUCE_SCATTER;
        if (len * ein <= ll_limit(k) && len * ein > 0) {
            mgk::coll::LLArgs l;
            memset(&l, 0, sizeof(l));
            l.in = in;
            l.out = wants_out ? out : nullptr;
            l.bytes = len * ein;
            l.reduce = 1;
            l.scale = scale;
            l.in_dtype = in_dtype;
            l.out_dtype = out_dtype;
            l.op = op;
            const uint32_t others = ((1u << n) - 1) & ~(1u << m_rank);
            if (kind == ReduceKind::AllReduce) {
                l.send_mask = l.recv_mask = others;
                l.self = 1;
            } else if (kind == ReduceKind::ReduceScatter) {
                l.send_mask = l.recv_mask = others;
                l.self = 1;
                for (uint32_t q = 0; q < n; ++q)
                    l.send_off[q] = static_cast<int64_t>(q * len * ein);
            } else {
                l.tokens = 1;
                if (m_rank == root) {
                    l.recv_mask = others;
                    l.self = 1;
                } else {
                    l.send_mask = 1u << root;
                }
            }
            return ll_launch(l, stream);
        }
    }

    // Ranks of one process: single pass on the buffers as they are.
    if (m_xchg && m_direct &&
        exchange_fits(in, len * ein * (kind == ReduceKind::ReduceScatter ? n : 1), wants_out ? out : nullptr, len * eout)) {
        if (kind == ReduceKind::AllReduce && (len * ein > m_oneshot_bytes || !m_oneshot_first))
            return exchange_launch(mgk::coll::DIRECT_ALL_REDUCE, in, len * ein, true, out, len * eout, true, len,
                                   in_dtype, out_dtype, scale, op, 0, stream);
        if (kind == ReduceKind::ReduceScatter)
            return exchange_launch(mgk::coll::DIRECT_REDUCE_SCATTER, in, len * ein * n, true, out, len * eout, false,
                                   len, in_dtype, out_dtype, scale, op, 0, stream);
        if (kind == ReduceKind::Reduce)
            return exchange_launch(mgk::coll::DIRECT_REDUCE, in, len * ein, true, wants_out ? out : nullptr,
                                   len * eout, true, len, in_dtype, out_dtype, scale, op, root, stream);
    }

    // Buffers inside the symmetric heap (at the same offset on every rank, which is what
    // sym_alloc gives) need no staging: single-pass kernels read and write the peers directly.
    if (m_direct && n > 1 && len * ein > m_oneshot_bytes) {
        if (kind == ReduceKind::AllReduce && aligned_heap(in, len * ein) && aligned_heap(out, len * eout))
            return direct_launch(mgk::coll::DIRECT_ALL_REDUCE, in, out, len, in_dtype, out_dtype, scale, op, stream);
        if (kind == ReduceKind::ReduceScatter && aligned_heap(in, len * ein * n) && (len * ein) % 16 == 0 &&
            (reinterpret_cast<uintptr_t>(out) & 15) == 0)
            return direct_launch(mgk::coll::DIRECT_REDUCE_SCATTER, in, out, len, in_dtype, out_dtype, scale, op,
                                 stream);
    }

    if (kind == ReduceKind::ReduceScatter) {
        // `len` is the per-rank result length; slice j of the input starts at j*len
        for (size_t off = 0; off < len; off += se_max) {
            const size_t se = std::min(se_max, len - off);
            a.c = common_args();
            const size_t ws = workspace_off();
            a.in = inb + off * ein;
            a.out = outb + off * eout;
            a.slice_elems = se;
            a.len = se * n;
            a.in_pitch_elems = len;
            a.stage_off = ws;
            a.red_off = ws + n * round_up(se * ein, 16);
            a.one_shot = 0;
            a.out_is_slice = 1;
            MEGRAY_CHECK(check_cuda(mgk::coll::launch_reduce(a, pick_ctas(se * ein * n), 512, stream)));
            after_launch(stream);
            m_stats.algo_twoshot++;
        }
        return MEGRAY_OK;
    }

    // all_reduce / reduce: small messages in one shot, larger ones in two
    const size_t bytes = len * ein;
    const bool fits_oneshot = n * round_up(bytes, 16) + round_up(len * eout, 16) <= m_ws_bytes;
    if (kind == ReduceKind::AllReduce && bytes <= m_oneshot_bytes && fits_oneshot) {
        a.c = common_args();
        const size_t ws = workspace_off();
        a.in = in;
        a.out = out;
        a.len = len;
        a.slice_elems = len;
        a.in_pitch_elems = len;
        a.stage_off = ws;
        a.red_off = ws + n * round_up(bytes, 16);
        a.one_shot = 1;
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_reduce(a, pick_ctas(bytes * n), 512, stream)));
        after_launch(stream);
        m_stats.algo_oneshot++;
        return MEGRAY_OK;
    }
    const size_t piece = se_max * n;
    for (size_t off = 0; off < len; off += piece) {
        const size_t this_len = std::min(piece, len - off);
        const size_t se = round_up((this_len + n - 1) / n, 16);
        a.c = common_args();
        const size_t ws = workspace_off();
        a.in = inb + off * ein;
        a.out = wants_out ? outb + off * eout : nullptr;
        a.len = this_len;
        a.slice_elems = se;
        a.in_pitch_elems = se;
        a.stage_off = ws;
        a.red_off = ws + n * round_up(se * ein, 16);
        a.one_shot = 0;
        a.out_is_slice = 0;
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_reduce(a, pick_ctas(this_len * ein), 512, stream)));
        after_launch(stream);
        m_stats.algo_twoshot++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::all_reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                   ReduceOp op, std::shared_ptr<Context> ctx) {
    if (dtype == MEGRAY_CHAR || dtype >= MEGRAY_DTYPE_COUNT || op >= MEGRAY_REDUCEOP_COUNT)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    TraceScope trace("all_reduce", len * get_dtype_size(dtype), m_rank);
    return reduce_impl(ReduceKind::AllReduce, sendbuff, recvbuff, len, dtype, dtype, 1.0f, op, 0,
                       stream);
}

Status NvlCommunicator::all_reduce_scaled(const void* sendbuff, void* recvbuff, size_t len,
                                          DType in_dtype, DType out_dtype, float scale,
                                          ReduceOp op, std::shared_ptr<Context> ctx) {
    if (!is_float(in_dtype) || !is_float(out_dtype) || op >= MEGRAY_REDUCEOP_COUNT)
        return MEGRAY_INVALID_ARGUMENT;
    if ((in_dtype == MEGRAY_FLOAT64) != (out_dtype == MEGRAY_FLOAT64))
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    TraceScope trace("all_reduce_scaled", len * get_dtype_size(in_dtype), m_rank);
    return reduce_impl(ReduceKind::AllReduce, sendbuff, recvbuff, len, in_dtype, out_dtype, scale,
                       op, 0, stream);
}

Status NvlCommunicator::reduce_scatter(const void* sendbuff, void* recvbuff, size_t recvlen,
                                       DType dtype, ReduceOp op, std::shared_ptr<Context> ctx) {
    if (dtype == MEGRAY_CHAR || dtype >= MEGRAY_DTYPE_COUNT || op >= MEGRAY_REDUCEOP_COUNT)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    TraceScope trace("reduce_scatter", recvlen * get_dtype_size(dtype), m_rank);
    return reduce_impl(ReduceKind::ReduceScatter, sendbuff, recvbuff, recvlen, dtype, dtype, 1.0f,
                       op, 0, stream);
}

Status NvlCommunicator::reduce(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                               ReduceOp op, uint32_t root, std::shared_ptr<Context> ctx) {
    if (dtype == MEGRAY_CHAR || dtype >= MEGRAY_DTYPE_COUNT || op >= MEGRAY_REDUCEOP_COUNT ||
        root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    TraceScope trace("reduce", len * get_dtype_size(dtype), m_rank);
    return reduce_impl(ReduceKind::Reduce, sendbuff, recvbuff, len, dtype, dtype, 1.0f, op, root,
                       stream);
}

// ------------------------------------------------------------------ exchange family

Status NvlCommunicator::all_gather(const void* sendbuff, void* recvbuff, size_t sendlen,
                                   DType dtype, std::shared_ptr<Context> ctx) {
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    const size_t bytes = sendlen * get_dtype_size(dtype);
    TraceScope trace("all_gather", bytes, m_rank);
    m_stats.bytes += bytes;
    if (bytes == 0)
        return MEGRAY_OK;
    if (sendbuff == nullptr || recvbuff == nullptr)
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(sendbuff, bytes, recvbuff, bytes * m_nranks);
    if (bytes <= ll_limit(mgk::coll::DIRECT_ALL_GATHER)) {
        mgk::coll::LLArgs l;
        memset(&l, 0, sizeof(l));
        l.in = sendbuff;
        l.out = recvbuff;
        l.bytes = bytes;
        l.send_mask = l.recv_mask = ((1u << m_nranks) - 1) & ~(1u << m_rank);
        l.self = 1;
        for (uint32_t q = 0; q < m_nranks; ++q)
            l.recv_off[q] = static_cast<int64_t>(q * bytes);
        return ll_launch(l, stream);
    }
    if (m_xchg && m_direct && exchange_fits(sendbuff, bytes, recvbuff, bytes * m_nranks))
        return exchange_launch(mgk::coll::DIRECT_ALL_GATHER, sendbuff, bytes, false, recvbuff, bytes * m_nranks, true,
                               bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f, MEGRAY_SUM, 0, stream);
    if (m_direct && m_nranks > 1 && bytes > m_oneshot_bytes / m_nranks && aligned_heap(recvbuff, bytes * m_nranks) &&
        bytes % 16 == 0)
        return direct_launch(mgk::coll::DIRECT_ALL_GATHER, sendbuff, recvbuff, bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f,
                             MEGRAY_SUM, stream);
    const size_t cap = round_down(m_ws_bytes - 16, 16);
    for (size_t off = 0; off < bytes; off += cap) {
        const size_t piece = std::min(cap, bytes - off);
        ExchangeArgs a;
        memset(&a, 0, sizeof(a));
        a.c = common_args();
        a.pub_off = workspace_off();
        a.in = static_cast<const char*>(sendbuff) + off;
        a.out = static_cast<char*>(recvbuff) + off;
        a.chunk_bytes = piece;
        a.in_pitch = bytes;
        a.out_pitch = bytes;
        a.publish_chunks = 1;
        a.push_root = -1;
        a.pull_mask = (1u << m_nranks) - 1;
        for (uint32_t q = 0; q < m_nranks; ++q) {
            a.src_chunk[q] = 0;
            a.dst_chunk[q] = static_cast<int>(q);
            a.pull_bytes[q] = piece;
            a.push_chunk[q] = 0;
        }
        a.push_all = m_push_exchange && bytes <= kPushExchangeBytes &&
                     round_up(piece, 16) * m_nranks <= m_ws_bytes;
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, pick_ctas(piece * m_nranks), 512, stream)));
        after_launch(stream);
        m_stats.algo_copy++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::all_to_all(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                   std::shared_ptr<Context> ctx) {
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    const size_t bytes = len * get_dtype_size(dtype);
    TraceScope trace("all_to_all", bytes, m_rank);
    m_stats.bytes += bytes;
    if (bytes == 0)
        return MEGRAY_OK;
    if (sendbuff == nullptr || recvbuff == nullptr)
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(sendbuff, bytes * m_nranks, recvbuff, bytes * m_nranks);
    if (bytes <= ll_limit(mgk::coll::DIRECT_ALL_TO_ALL)) {
        mgk::coll::LLArgs l;
        memset(&l, 0, sizeof(l));
        l.in = sendbuff;
        l.out = recvbuff;
        l.bytes = bytes;
        l.send_mask = l.recv_mask = ((1u << m_nranks) - 1) & ~(1u << m_rank);
        l.self = 1;
        for (uint32_t q = 0; q < m_nranks; ++q)
            l.send_off[q] = l.recv_off[q] = static_cast<int64_t>(q * bytes);
        return ll_launch(l, stream);
    }
    if (m_xchg && m_direct && exchange_fits(sendbuff, bytes * m_nranks, recvbuff, bytes * m_nranks))
        return exchange_launch(mgk::coll::DIRECT_ALL_TO_ALL, sendbuff, bytes * m_nranks, false, recvbuff,
                               bytes * m_nranks, true, bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f, MEGRAY_SUM, 0, stream);
    if (m_direct && m_nranks > 1 && bytes > m_oneshot_bytes / m_nranks && aligned_heap(recvbuff, bytes * m_nranks) &&
        bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(sendbuff) & 15) == 0)
        return direct_launch(mgk::coll::DIRECT_ALL_TO_ALL, sendbuff, recvbuff, bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f,
                             MEGRAY_SUM, stream);
    const size_t cap = round_down(m_ws_bytes / m_nranks - 16, 16);
    for (size_t off = 0; off < bytes; off += cap) {
        const size_t piece = std::min(cap, bytes - off);
        ExchangeArgs a;
        memset(&a, 0, sizeof(a));
        a.c = common_args();
        a.pub_off = workspace_off();
        a.in = static_cast<const char*>(sendbuff) + off;
        a.out = static_cast<char*>(recvbuff) + off;
        a.chunk_bytes = piece;
        a.in_pitch = bytes;
        a.out_pitch = bytes;
        a.publish_chunks = static_cast<int>(m_nranks);
        a.push_root = -1;
        a.pull_mask = (1u << m_nranks) - 1;
        for (uint32_t q = 0; q < m_nranks; ++q) {
            a.src_chunk[q] = static_cast<int>(m_rank);
            a.dst_chunk[q] = static_cast<int>(q);
            a.pull_bytes[q] = piece;
            a.push_chunk[q] = static_cast<int>(q);
        }
        a.push_all = m_push_exchange && bytes <= kPushExchangeBytes;
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, pick_ctas(piece * m_nranks), 512, stream)));
        after_launch(stream);
        m_stats.algo_copy++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::broadcast(const void* sendbuff, void* recvbuff, size_t len, DType dtype,
                                  uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    const size_t bytes = len * get_dtype_size(dtype);
    TraceScope trace("broadcast", bytes, m_rank);
    m_stats.bytes += bytes;
    if (bytes == 0)
        return MEGRAY_OK;
    if (recvbuff == nullptr || (m_rank == root && sendbuff == nullptr))
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(m_rank == root ? sendbuff : nullptr, bytes, recvbuff, bytes);
    if (bytes <= ll_limit(mgk::coll::DIRECT_BROADCAST)) {
        mgk::coll::LLArgs l;
        memset(&l, 0, sizeof(l));
        l.in = m_rank == root ? sendbuff : nullptr;
        l.out = recvbuff;
        l.bytes = bytes;
        l.tokens = 1;
        if (m_rank == root) {
            l.send_mask = ((1u << m_nranks) - 1) & ~(1u << m_rank);
            l.self = sendbuff != recvbuff ? 1 : 0;
        } else {
            l.recv_mask = 1u << root;
        }
        return ll_launch(l, stream);
    }
    if (m_xchg && m_direct && exchange_fits(m_rank == root ? sendbuff : nullptr, bytes, recvbuff, bytes))
        // (in the loads-only form the peers read the root's input themselves)
        return exchange_launch(mgk::coll::DIRECT_BROADCAST, m_rank == root ? sendbuff : nullptr, bytes,
                               m_bcast_pull && bytes >= m_bcast_pull_min, recvbuff, bytes, true, bytes, MEGRAY_UINT8,
                               MEGRAY_UINT8, 1.0f, MEGRAY_SUM, root, stream);
    const uint32_t n = m_nranks;
    const bool two_step = bytes > m_oneshot_bytes && n > 2;
    // one step: everyone loads the whole piece from the root's pub buffer
    // two steps: the root pushes slice j to peer j, then everyone loads all slices
    const size_t cap = two_step ? round_down(m_ws_bytes - 16, 16) * n : round_down(m_ws_bytes - 16, 16);
    for (size_t off = 0; off < bytes; off += cap) {
        const size_t piece = std::min(cap, bytes - off);
        ExchangeArgs a;
        memset(&a, 0, sizeof(a));
        a.c = common_args();
        a.pub_off = workspace_off();
        a.in = m_rank == root ? static_cast<const char*>(sendbuff) + off : nullptr;
        a.out = static_cast<char*>(recvbuff) + off;
        if (two_step) {
            const size_t sb = round_up((piece + n - 1) / n, 16);
            a.chunk_bytes = sb;
            a.in_pitch = sb;
            a.out_pitch = sb;
            a.push_root = static_cast<int>(root);
            a.pull_mask = (1u << n) - 1;
            for (uint32_t q = 0; q < n; ++q) {
                const size_t s0 = static_cast<size_t>(q) * sb;
                a.src_chunk[q] = 0;
                a.dst_chunk[q] = static_cast<int>(q);
                a.pull_bytes[q] = s0 >= piece ? 0 : std::min(sb, piece - s0);
            }
        } else {
            a.chunk_bytes = piece;
            a.in_pitch = piece;
            a.out_pitch = piece;
            a.publish_chunks = m_rank == root ? 1 : 0;
            a.push_root = -1;
            a.pull_mask = 1u << root;
            a.pull_bytes[root] = piece;
        }
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, pick_ctas(piece), 512, stream)));
        after_launch(stream);
        m_stats.algo_copy++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::gather(const void* sendbuff, void* recvbuff, size_t sendlen, DType dtype,
                               uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    const size_t bytes = sendlen * get_dtype_size(dtype);
    TraceScope trace("gather", bytes, m_rank);
    m_stats.bytes += bytes;
    if (bytes == 0)
        return MEGRAY_OK;
    if (sendbuff == nullptr || (m_rank == root && recvbuff == nullptr))
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(sendbuff, bytes, m_rank == root ? recvbuff : nullptr, bytes * m_nranks);
    if (bytes <= ll_limit(mgk::coll::DIRECT_GATHER)) {
        mgk::coll::LLArgs l;
        memset(&l, 0, sizeof(l));
        l.in = sendbuff;
        l.out = m_rank == root ? recvbuff : nullptr;
        l.bytes = bytes;
        l.tokens = 1;
        if (m_rank == root) {
            l.recv_mask = ((1u << m_nranks) - 1) & ~(1u << m_rank);
            l.self = 1;
            for (uint32_t q = 0; q < m_nranks; ++q)
                l.recv_off[q] = static_cast<int64_t>(q * bytes);
        } else {
            l.send_mask = 1u << root;
        }
        return ll_launch(l, stream);
    }
    if (m_xchg && m_direct && exchange_fits(sendbuff, bytes, m_rank == root ? recvbuff : nullptr, bytes * m_nranks))
        return exchange_launch(mgk::coll::DIRECT_GATHER, sendbuff, bytes, false, m_rank == root ? recvbuff : nullptr,
                               bytes * m_nranks, true, bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f, MEGRAY_SUM, root,
                               stream);
    const size_t cap = round_down(m_ws_bytes - 16, 16);
    for (size_t off = 0; off < bytes; off += cap) {
        const size_t piece = std::min(cap, bytes - off);
        ExchangeArgs a;
        memset(&a, 0, sizeof(a));
        a.c = common_args();
        a.pub_off = workspace_off();
        a.in = static_cast<const char*>(sendbuff) + off;
        a.out = m_rank == root ? static_cast<char*>(recvbuff) + off : nullptr;
        a.chunk_bytes = piece;
        a.in_pitch = bytes;
        a.out_pitch = bytes;
        a.publish_chunks = 1;
        a.push_root = -1;
        a.pull_mask = m_rank == root ? (1u << m_nranks) - 1 : 0;
        for (uint32_t q = 0; q < m_nranks; ++q) {
            a.src_chunk[q] = 0;
            a.dst_chunk[q] = static_cast<int>(q);
            a.pull_bytes[q] = piece;
        }
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, pick_ctas(piece * m_nranks), 512, stream)));
        after_launch(stream);
        m_stats.algo_copy++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::scatter(const void* sendbuff, void* recvbuff, size_t recvlen, DType dtype,
                                uint32_t root, std::shared_ptr<Context> ctx) {
    if (root >= m_nranks)
        return MEGRAY_INVALID_ARGUMENT;
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    const size_t bytes = recvlen * get_dtype_size(dtype);
    TraceScope trace("scatter", bytes, m_rank);
    m_stats.bytes += bytes;
    if (bytes == 0)
        return MEGRAY_OK;
    if (recvbuff == nullptr || (m_rank == root && sendbuff == nullptr))
        return MEGRAY_INVALID_ARGUMENT;
    set_guard(m_rank == root ? sendbuff : nullptr, bytes * m_nranks, recvbuff, bytes);
    if (bytes <= ll_limit(mgk::coll::DIRECT_SCATTER)) {
        mgk::coll::LLArgs l;
        memset(&l, 0, sizeof(l));
        l.in = m_rank == root ? sendbuff : nullptr;
        l.out = recvbuff;
        l.bytes = bytes;
        l.tokens = 1;
        if (m_rank == root) {
            l.send_mask = ((1u << m_nranks) - 1) & ~(1u << m_rank);
            l.self = 1;
            for (uint32_t q = 0; q < m_nranks; ++q)
                l.send_off[q] = static_cast<int64_t>(q * bytes);
        } else {
            l.recv_mask = 1u << root;
        }
        return ll_launch(l, stream);
    }
    if (m_xchg && m_direct && exchange_fits(m_rank == root ? sendbuff : nullptr, bytes * m_nranks, recvbuff, bytes))
        return exchange_launch(mgk::coll::DIRECT_SCATTER, m_rank == root ? sendbuff : nullptr, bytes * m_nranks, false,
                               recvbuff, bytes, true, bytes, MEGRAY_UINT8, MEGRAY_UINT8, 1.0f, MEGRAY_SUM, root,
                               stream);
    const size_t cap = round_down(m_ws_bytes / m_nranks - 16, 16);
    for (size_t off = 0; off < bytes; off += cap) {
        const size_t piece = std::min(cap, bytes - off);
        ExchangeArgs a;
        memset(&a, 0, sizeof(a));
        a.c = common_args();
        a.pub_off = workspace_off();
        a.in = m_rank == root ? static_cast<const char*>(sendbuff) + off : nullptr;
        a.out = static_cast<char*>(recvbuff) + off;
        a.chunk_bytes = piece;
        a.in_pitch = bytes;
        a.out_pitch = bytes;
        a.publish_chunks = m_rank == root ? static_cast<int>(m_nranks) : 0;
        a.push_root = -1;
        a.pull_mask = 1u << root;
        a.src_chunk[root] = static_cast<int>(m_rank);
        a.dst_chunk[root] = 0;
        a.pull_bytes[root] = piece;
        MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, pick_ctas(piece * m_nranks), 512, stream)));
        after_launch(stream);
        m_stats.algo_copy++;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::stream_barrier(std::shared_ptr<Context> ctx) {
    cudaStream_t stream;
    MEGRAY_CHECK(begin(ctx, &stream));
    set_guard(nullptr, 0, nullptr, 0);
    ExchangeArgs a;
    memset(&a, 0, sizeof(a));
    a.c = common_args();
    a.pub_off = workspace_off();
    a.push_root = -1;
    MEGRAY_CHECK(check_cuda(mgk::coll::launch_exchange(a, 1, 32, stream)));
    after_launch(stream);
    return MEGRAY_OK;
}

// ------------------------------------------------------------------ point to point (NCCL)
// send / recv run as NCCL point-to-point calls.  In the ordinary mode they go straight onto the
// caller's stream.  With set_p2p_async(true) they run on a stream of the communicator's own.  That
// stream first waits for the work already on the caller's stream (the data to send is final, the
// buffer to receive into is free) and the caller's stream then waits for the transfer, so the
// calls keep the interface's meaning: enqueued on the context's stream, complete in stream order;
// but the second wait is left out until p2p_join(): kernels enqueued on the
// caller's stream in between (native collectives included) run at the same time as the transfer.

Status NvlCommunicator::p2p_fork(cudaStream_t user) {
    if (m_p2p_stream == nullptr) {
        CUDA_CHECK(cudaStreamCreateWithFlags(&m_p2p_stream, cudaStreamNonBlocking));
        CUDA_CHECK(cudaEventCreateWithFlags(&m_p2p_fork, cudaEventDisableTiming));
        CUDA_CHECK(cudaEventCreateWithFlags(&m_p2p_done, cudaEventDisableTiming));
    }
    for (cudaStream_t s : m_p2p_users)
        if (s == user)
            return MEGRAY_OK;  // this group already waits for that stream
    CUDA_CHECK(cudaEventRecord(m_p2p_fork, user));
    CUDA_CHECK(cudaStreamWaitEvent(m_p2p_stream, m_p2p_fork, 0));
    m_p2p_users.push_back(user);
    return MEGRAY_OK;
}

Status NvlCommunicator::p2p_finish() {
    CUDA_CHECK(cudaEventRecord(m_p2p_done, m_p2p_stream));
    if (m_p2p_async) {
        m_p2p_pending = true;
    } else {
        for (cudaStream_t s : m_p2p_users)
            CUDA_CHECK(cudaStreamWaitEvent(s, m_p2p_done, 0));
    }
    m_p2p_users.clear();
    return MEGRAY_OK;
}

Status NvlCommunicator::p2p_join(std::shared_ptr<Context> ctx) {
    if (!ctx || ctx->type() != MEGRAY_CTX_CUDA)
        return MEGRAY_INVALID_ARGUMENT;
    if (m_p2p_pending) {
        CUDA_CHECK(cudaStreamWaitEvent(static_cast<CudaContext*>(ctx.get())->get_stream(), m_p2p_done, 0));
        m_p2p_pending = false;
    }
    return MEGRAY_OK;
}

Status NvlCommunicator::p2p_call(bool is_send, void* buf, size_t size, uint32_t rank,
                                 const std::shared_ptr<Context>& ctx) {
#ifdef MEGRAY_WITH_NCCL
    if (!m_p2p)
        return MEGRAY_NOT_IMPLEMENTED;
    if (!ctx || ctx->type() != MEGRAY_CTX_CUDA)
        return MEGRAY_INVALID_ARGUMENT;
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    m_stats.calls++;
    m_stats.bytes += size;
    if (!m_p2p_async && !m_p2p_pending && m_p2p_users.empty()) {
        // Joined at once, the transfer would run in the caller's stream order anyway: enqueue it
        // there (as the reference does, src/nccl/communicator.cpp:66-88) and save the fork / join events.
        return is_send ? m_p2p->send(buf, size, MEGRAY_CHAR, rank, ctx) : m_p2p->recv(buf, size, MEGRAY_CHAR, rank, ctx);
    }
    MEGRAY_CHECK(p2p_fork(static_cast<CudaContext*>(ctx.get())->get_stream()));
    if (!m_p2p_ctx)
        m_p2p_ctx = CudaContext::make(m_p2p_stream);
    const Status s = is_send ? m_p2p->send(buf, size, MEGRAY_CHAR, rank, m_p2p_ctx)
                             : m_p2p->recv(buf, size, MEGRAY_CHAR, rank, m_p2p_ctx);
    if (s != MEGRAY_OK) {
        m_p2p_users.clear();
        return s;
    }
    return m_p2p_grouping ? MEGRAY_OK : p2p_finish();
#else
    return MEGRAY_NOT_IMPLEMENTED;
#endif
}

Status NvlCommunicator::_send(const void* sendbuff, size_t size, uint32_t rank,
                              std::shared_ptr<Context> ctx) {
    return p2p_call(true, const_cast<void*>(sendbuff), size, rank, ctx);
}

Status NvlCommunicator::_recv(void* recvbuf, size_t size, uint32_t rank,
                              std::shared_ptr<Context> ctx) {
    return p2p_call(false, recvbuf, size, rank, ctx);
}

Status NvlCommunicator::group_start() {
#ifdef MEGRAY_WITH_NCCL
    // native collectives are single launches and ignore grouping; p2p is batched by NCCL
    if (m_p2p) {
        m_p2p_grouping = true;
        return m_p2p->group_start();
    }
#endif
    return MEGRAY_OK;
}

Status NvlCommunicator::group_end() {
#ifdef MEGRAY_WITH_NCCL
    if (m_p2p) {
        m_p2p_grouping = false;
        const Status s = m_p2p->group_end();
        if (s != MEGRAY_OK) {
            m_p2p_users.clear();
            return s;
        }
        return m_p2p_users.empty() ? MEGRAY_OK : p2p_finish();
    }
#endif
    return MEGRAY_OK;
}

// ------------------------------------------------------------------ state

void NvlCommunicator::abort() {
    Communicator::abort();
#ifdef MEGRAY_WITH_NCCL
    if (m_p2p)
        m_p2p->abort();
#endif
}

Status NvlCommunicator::status() {
    if (m_aborted.load())
        return MEGRAY_ABORTED;
    if (m_status_host != nullptr && *m_status_host != 0)
        adopt_device_status();
    return m_error;
}

CommStats NvlCommunicator::stats() { return m_stats; }

// ------------------------------------------------------------------ symmetric allocator

void* NvlCommunicator::sym_alloc(size_t bytes, size_t* offset_out) {
    if (!m_ready || bytes == 0)
        return nullptr;
    const size_t at = round_up(m_user_top, 1024);
    if (at + bytes > m_heap.bytes()) {
        MEGRAY_ERROR("symmetric heap exhausted: %zu bytes wanted, %zu free (MEGRAY_HEAP_MB=%lld)", bytes,
                     m_heap.bytes() - at, static_cast<long long>(global_options().heap_mb));
        return nullptr;
    }
    m_allocs.push_back(m_user_top);
    m_user_top = at + bytes;
    if (offset_out != nullptr)
        *offset_out = at;
    return m_heap.local() + at;
}

Status NvlCommunicator::sym_free(void* ptr) {
    if (!in_heap(ptr, 1))
        return MEGRAY_INVALID_ARGUMENT;
    const size_t off = static_cast<size_t>(static_cast<char*>(ptr) - m_heap.local());
    while (!m_allocs.empty()) {
        const size_t prev_top = m_allocs.back();
        m_allocs.pop_back();
        const size_t at = round_up(prev_top, 1024);
        m_user_top = prev_top;
        // counter blocks in the released range start from zero for their next owner
        m_fused_calls.erase(m_fused_calls.lower_bound(at), m_fused_calls.end());
        if (at == off)
            return MEGRAY_OK;
        if (at < off)
            break;
    }
    return MEGRAY_INVALID_ARGUMENT;
}

void* NvlCommunicator::peer_ptr(void* ptr, uint32_t peer) {
    if (peer >= m_nranks || !in_heap(ptr, 1))
        return nullptr;
    return m_heap.base(peer) + (static_cast<char*>(ptr) - m_heap.local());
}

bool NvlCommunicator::in_heap(const void* ptr, size_t bytes) {
    if (!m_ready || ptr == nullptr)
        return false;
    const char* p = static_cast<const char*>(ptr);
    return p >= m_heap.local() && p + bytes <= m_heap.local() + m_heap.bytes();
}

// ------------------------------------------------------------------ registered user buffers

namespace {
// What the ranks tell each other about the buffers they register in one call.
struct RegInfo {
    int32_t pid;
    int32_t device;
    int32_t ok;       // 0: this rank could not export its buffer
    int32_t pad;
    uint64_t ptr;     // the buffer as its owner addresses it
    uint64_t bytes;
    uint64_t offset;  // distance of `ptr` from the start of its allocation (what an IPC handle maps)
    cudaIpcMemHandle_t handle;
};
}  // namespace

bool NvlCommunicator::peer_view(const void* p, size_t bytes, char** base, size_t* heap_off) {
    if (!m_ready || p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) != 0)
        return false;
    const char* c = static_cast<const char*>(p);
    if (in_heap(p, bytes)) {
        const size_t off = static_cast<size_t>(c - m_heap.local());
        for (uint32_t q = 0; q < m_nranks; ++q)
            base[q] = m_heap.base(q) + off;
        *heap_off = off;
        return true;
    }
    for (const Registration& r : m_regs) {
        if (c >= r.local && c + bytes <= r.local + r.bytes) {
            const size_t off = static_cast<size_t>(c - r.local);
            for (uint32_t q = 0; q < m_nranks; ++q)
                base[q] = r.peer[q] + off;
            *heap_off = SIZE_MAX;
            return true;
        }
    }
    return false;
}

void NvlCommunicator::drop_registration(Registration& r) {
    for (void* b : r.ipc_bases)
        cudaIpcCloseMemHandle(b);
    r.ipc_bases.clear();
}

Status NvlCommunicator::register_buffer(void* ptr, size_t bytes) {
    if (!m_ready)
        return MEGRAY_INVALID_USAGE;
    // A bad argument on one rank must not leave the others waiting in the exchange below: it is
    // reported to them as "this rank could not export its buffer", and every rank falls back.
    const bool bad_arg = ptr == nullptr || bytes == 0;
    if (m_ipc != nullptr) {
        // Ranks in separate processes export allocations of moderate size on first use anyway;
        // registering exports one of any size and returns when every peer has mapped it.
        if (bad_arg)
            return MEGRAY_INVALID_ARGUMENT;
        if (in_heap(ptr, bytes))
            return MEGRAY_OK;
        // (waits until every peer has mapped it: afterwards calls of any size on it are single-pass)
        return m_ipc->register_range(ptr, bytes, global_options().timeout_ms > 0 ? global_options().timeout_ms : 30000);
    }
    const drv::Api* api = drv::api();
    std::vector<RegInfo> all(m_nranks);
    RegInfo mine;
    memset(&mine, 0, sizeof(mine));
    mine.pid = static_cast<int32_t>(getpid());
    mine.device = m_heap.device();
    mine.ptr = reinterpret_cast<uint64_t>(ptr);
    mine.bytes = bytes;
    mine.ok = 1;
    CUdeviceptr alloc_base = 0;
    size_t alloc_size = 0;
    if (bad_arg || api == nullptr ||
        api->MemGetAddressRange(&alloc_base, &alloc_size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS ||
        reinterpret_cast<CUdeviceptr>(ptr) + bytes > alloc_base + alloc_size) {
        mine.ok = 0;  // not one device allocation
    } else {
        mine.offset = reinterpret_cast<CUdeviceptr>(ptr) - alloc_base;
        // only needed by peers in other processes; memory without an IPC handle (virtual memory
        // management allocations) still works between ranks of one process
        if (cudaIpcGetMemHandle(&mine.handle, reinterpret_cast<void*>(alloc_base)) != cudaSuccess) {
            (void)cudaGetLastError();
            mine.ok = 2;  // usable inside this process only
        }
    }
    MEGRAY_CHECK(m_client->allgather(&mine, all.data(), sizeof(RegInfo)));
    bool usable = true;
    for (uint32_t q = 0; q < m_nranks; ++q) {
        if (all[q].ok == 0)
            usable = false;
        if (all[q].ok == 2 && all[q].pid != mine.pid)
            usable = false;
        if (all[q].bytes != bytes)
            usable = false;
    }
    Registration r;
    r.local = static_cast<char*>(ptr);
    r.bytes = bytes;
    int32_t opened_ok = usable ? 1 : 0;
    if (usable) {
        for (uint32_t q = 0; q < m_nranks && opened_ok; ++q) {
            if (q == m_rank) {
                r.peer[q] = r.local;
            } else if (all[q].pid == mine.pid) {
                // the same address space: the peer's address is valid here once peer access is on
                cudaError_t e = cudaDeviceEnablePeerAccess(all[q].device, 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
                    opened_ok = 0;
                (void)cudaGetLastError();
                r.peer[q] = reinterpret_cast<char*>(all[q].ptr);
            } else {
                void* base = nullptr;
                cudaError_t e = cudaIpcOpenMemHandle(&base, all[q].handle, cudaIpcMemLazyEnablePeerAccess);
                if (e != cudaSuccess) {
                    (void)cudaGetLastError();
                    opened_ok = 0;
                } else {
                    r.ipc_bases.push_back(base);
                    r.peer[q] = static_cast<char*>(base) + all[q].offset;
                }
            }
        }
    }
    // all or nothing: a rank that could not map a peer makes everyone fall back
    std::vector<int32_t> oks(m_nranks);
    MEGRAY_CHECK(m_client->allgather(&opened_ok, oks.data(), sizeof(int32_t)));
    for (uint32_t q = 0; q < m_nranks; ++q)
        if (!oks[q])
            usable = false;
    if (!usable) {
        drop_registration(r);
        MEGRAY_INFO("register_buffer: %p (%zu bytes) stays on the staged paths", ptr, bytes);
        return bad_arg ? MEGRAY_INVALID_ARGUMENT : MEGRAY_NOT_IMPLEMENTED;
    }
    m_regs.push_back(std::move(r));
    return MEGRAY_OK;
}

Status NvlCommunicator::deregister_buffer(void* ptr) {
    if (!m_ready)
        return MEGRAY_INVALID_ARGUMENT;
    // peers may still be reading or writing this buffer from their last kernel
    cudaDeviceSynchronize();
    MEGRAY_CHECK(m_client->barrier());
    if (m_ipc != nullptr)
        return MEGRAY_OK;  // (exports stay: the memory may be used again)
    for (size_t i = 0; i < m_regs.size(); ++i) {
        if (m_regs[i].local == static_cast<char*>(ptr)) {
            drop_registration(m_regs[i]);
            m_regs.erase(m_regs.begin() + static_cast<long>(i));
            return MEGRAY_OK;
        }
    }
    return MEGRAY_INVALID_ARGUMENT;
}

}  // namespace MegRay
