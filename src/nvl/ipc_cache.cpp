#include "nvl/ipc_cache.h"

#include <stdlib.h>
#include <string.h>
#include <unistd.h>

#include <chrono>

#include "megray/debug.h"
#include "nvl/cuda_driver.h"

namespace MegRay {

namespace {
std::atomic<uint32_t> g_region_counter{0};
}

IpcCache::~IpcCache() {
    if (m_helper.joinable()) {
        {
            std::lock_guard<std::mutex> lk(m_mu);
            m_stop.store(true);
            m_kick = true;
        }
        m_cv.notify_all();
        m_helper.join();
    }
    for (auto& per_rank : m_mappings)
        for (void* base : per_rank)
            if (base != nullptr)
                cudaIpcCloseMemHandle(base);
    for (void* b : m_bounce)
        if (b != nullptr)
            cudaFree(b);
    if (m_stream != nullptr)
        cudaStreamDestroy(m_stream);
    if (m_table_dev != nullptr)
        cudaFree(m_table_dev);
    (void)cudaGetLastError();
}

bool IpcCache::init(Client& client, uint32_t nranks, uint32_t rank, int device) {
    m_nranks = nranks;
    m_rank = rank;
    m_device = device;
    if (const char* v = getenv("MEGRAY_IPC_AUTO_MAX_MB"))
        m_auto_max = static_cast<size_t>(atoll(v)) << 20;
    // rank 0 names and creates the region; the others attach
    char name[64];
    memset(name, 0, sizeof(name));
    if (rank == 0)
        snprintf(name, sizeof(name), "/megray_ipc_%d_%u", static_cast<int>(getpid()), g_region_counter.fetch_add(1));
    int32_t mine = 1;
    const size_t slot_bytes = (sizeof(RankLog) + 4095) / 4096 * 4096;
    if (rank == 0) {
        m_region = host::SharedRegion::create(name, nranks, slot_bytes, 0, false);
        if (!m_region)
            mine = 0;
        else
            for (uint32_t q = 0; q < nranks; ++q) {
                log(q)->count.store(0, std::memory_order_relaxed);
                for (auto& a : log(q)->imported_from)
                    a.store(0, std::memory_order_relaxed);
            }
    }
    if (client.broadcast(name, name, sizeof(name), 0) != MEGRAY_OK)
        return false;
    if (rank != 0) {
        m_region = host::SharedRegion::attach(name, false, 10000);
        if (!m_region)
            mine = 0;
    }
    if (mine && drv::api() == nullptr)
        mine = 0;
    if (mine) {
        const size_t table_bytes = static_cast<size_t>(nranks) * kMaxExports * sizeof(uint64_t);
        if (cudaMalloc(reinterpret_cast<void**>(&m_table_dev), table_bytes) != cudaSuccess ||
            cudaMemset(m_table_dev, 0, table_bytes) != cudaSuccess ||
            cudaStreamCreateWithFlags(&m_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaDeviceSynchronize() != cudaSuccess) {
            (void)cudaGetLastError();
            mine = 0;
        }
    }
    std::vector<int32_t> all(nranks, 0);
    if (client.allgather(&mine, all.data(), sizeof(int32_t)) != MEGRAY_OK)
        return false;
    for (uint32_t q = 0; q < nranks; ++q)
        if (!all[q])
            return false;
    m_imported.assign(nranks, 0);
    m_mappings.assign(nranks, std::vector<void*>());
    // Every rank exports its two bounce buffers now and maps everybody else's before any collective
    // runs.  A buffer of a call stands in for memory the peers have not mapped (yet); and the
    // first mapping of a peer's memory switches on peer access to its device, which touches every
    // allocation of this context and is best done while the devices are idle.
    {
        m_bounce_bytes = m_auto_max + (2u << 20);
        uint64_t word = 0;
        int32_t fine = 1;
        for (int i = 0; i < 2 && fine; ++i)
            fine = cudaMalloc(&m_bounce[i], m_bounce_bytes) == cudaSuccess && resolve(m_bounce[i], m_bounce_bytes, &word, true) ? 1 : 0;
        (void)cudaGetLastError();
        if (client.allgather(&fine, all.data(), sizeof(int32_t)) != MEGRAY_OK)
            return false;
        for (uint32_t q = 0; q < nranks; ++q)
            fine = fine && all[q] != 0;
        if (fine) {
            import_new();  // (everybody's two entries are in the logs: the allgather came after the exports)
            for (uint32_t q = 0; q < nranks; ++q)
                if (q != rank && m_imported[q] < 2)
                    fine = 0;
        }
        if (client.allgather(&fine, all.data(), sizeof(int32_t)) != MEGRAY_OK)
            return false;
        for (uint32_t q = 0; q < nranks; ++q)
            if (!all[q])
                return false;
    }
    m_helper = std::thread([this] { helper_main(); });
    return true;
}

bool IpcCache::resolve(const void* p, size_t bytes, uint64_t* word, bool any_size) {
    const drv::Api* api = drv::api();
    if (api == nullptr || p == nullptr)
        return false;
    unsigned int mem_type = 0;
    int ordinal = -1;
    int legacy = 0;
    CUdeviceptr start = 0;
    size_t size = 0;
    unsigned long long buffer_id = 0;
    CUpointer_attribute attrs[6] = {CU_POINTER_ATTRIBUTE_MEMORY_TYPE,
                                    CU_POINTER_ATTRIBUTE_DEVICE_ORDINAL,
                                    CU_POINTER_ATTRIBUTE_IS_LEGACY_CUDA_IPC_CAPABLE,
                                    CU_POINTER_ATTRIBUTE_RANGE_START_ADDR,
                                    CU_POINTER_ATTRIBUTE_RANGE_SIZE,
                                    CU_POINTER_ATTRIBUTE_BUFFER_ID};
    void* vals[6] = {&mem_type, &ordinal, &legacy, &start, &size, &buffer_id};
    const CUdeviceptr at = reinterpret_cast<CUdeviceptr>(p);
    if (api->PointerGetAttributes(6, attrs, vals, at) != CUDA_SUCCESS)
        return false;
    if (mem_type != CU_MEMORYTYPE_DEVICE || ordinal != m_device || legacy == 0 || at < start || at + bytes > start + size)
        return false;
    auto it = m_known.find(start);
    if (it != m_known.end() && it->second.buffer_id == buffer_id && it->second.size == size) {
        *word = encode(it->second.entry, at - start);
        return true;
    }
    if (size > m_auto_max && !any_size)
        return false;
    RankLog* mine = log(m_rank);
    const uint32_t entry = mine->count.load(std::memory_order_relaxed);
    if (entry >= kMaxExports)
        return false;
    ExportSlot& s = mine->slots[entry];
    memset(&s, 0, sizeof(s));
    if (cudaIpcGetMemHandle(&s.handle, reinterpret_cast<void*>(start)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    s.buffer_id = buffer_id;
    s.base = start;
    s.size = size;
    s.pid = static_cast<int32_t>(getpid());
    s.device = m_device;
    s.supersedes = it != m_known.end() ? it->second.entry : ~0u;
    mine->count.store(entry + 1, std::memory_order_release);
    m_known[start] = Known{buffer_id, size, entry};
    ++m_exports_made;
    {
        // peers tend to export at the same point of the program: have the helper look right away
        std::lock_guard<std::mutex> lk(m_mu);
        m_kick = true;
    }
    m_cv.notify_all();
    *word = encode(entry, at - start);
    return true;
}

bool IpcCache::entry_acked(uint32_t entry) {
    for (uint32_t q = 0; q < m_nranks; ++q)
        if (q != m_rank && log(q)->imported_from[m_rank].load(std::memory_order_acquire) <= entry)
            return false;
    return true;
}

bool IpcCache::mapped_everywhere(const void* p, size_t bytes) {
    const drv::Api* api = drv::api();
    if (api == nullptr || p == nullptr)
        return false;
    CUdeviceptr start = 0;
    size_t size = 0;
    unsigned long long buffer_id = 0;
    CUpointer_attribute attrs[3] = {CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, CU_POINTER_ATTRIBUTE_RANGE_SIZE,
                                    CU_POINTER_ATTRIBUTE_BUFFER_ID};
    void* vals[3] = {&start, &size, &buffer_id};
    const CUdeviceptr at = reinterpret_cast<CUdeviceptr>(p);
    if (api->PointerGetAttributes(3, attrs, vals, at) != CUDA_SUCCESS || at < start || at + bytes > start + size)
        return false;
    auto it = m_known.find(start);
    return it != m_known.end() && it->second.buffer_id == buffer_id && it->second.size == size &&
           entry_acked(it->second.entry);
}

bool IpcCache::resolve_mapped(const void* p, size_t bytes, uint64_t* word) {
    const drv::Api* api = drv::api();
    if (api == nullptr || p == nullptr)
        return false;
    CUdeviceptr start = 0;
    size_t size = 0;
    unsigned long long buffer_id = 0;
    CUpointer_attribute attrs[3] = {CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, CU_POINTER_ATTRIBUTE_RANGE_SIZE,
                                    CU_POINTER_ATTRIBUTE_BUFFER_ID};
    void* vals[3] = {&start, &size, &buffer_id};
    const CUdeviceptr at = reinterpret_cast<CUdeviceptr>(p);
    if (api->PointerGetAttributes(3, attrs, vals, at) != CUDA_SUCCESS || at < start || at + bytes > start + size)
        return false;
    auto it = m_known.find(start);
    if (it != m_known.end() && it->second.buffer_id == buffer_id && it->second.size == size) {
        if (!entry_acked(it->second.entry))
            return false;  // on its way
        *word = encode(it->second.entry, at - start);
        return true;
    }
    uint64_t unused = 0;
    (void)resolve(p, bytes, &unused);  // export it (unless too large or not exportable); usable once acknowledged
    return false;
}

Status IpcCache::register_range(const void* p, size_t bytes, int64_t timeout_ms) {
    uint64_t word = 0;
    if (!resolve(p, bytes, &word, true))
        return MEGRAY_NOT_IMPLEMENTED;
    const uint32_t entry = static_cast<uint32_t>(word >> 48);
    const auto until = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    while (!entry_acked(entry)) {
        if (std::chrono::steady_clock::now() > until)
            return MEGRAY_TIMEOUT;
        import_new();  // (the peers register theirs at the same point: map them here meanwhile)
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    // ... and until this rank has mapped what the peers have published so far (their registrations)
    import_new();
    return MEGRAY_OK;
}

bool IpcCache::import_new() {
    std::lock_guard<std::mutex> guard(m_import_mu);
    bool any = false;
    for (uint32_t q = 0; q < m_nranks; ++q) {
        if (q == m_rank)
            continue;
        RankLog* theirs = log(q);
        const uint32_t have = theirs->count.load(std::memory_order_acquire);
        while (m_imported[q] < have && !m_stop.load()) {
            const uint32_t e = m_imported[q];
            const ExportSlot& s = theirs->slots[e];
            uint64_t mapped = kImportFailed;
            void* to_close = nullptr;
            // (A superseded mapping - the owner freed that allocation and got the same address
            // again - stays open until this object goes: closing one waits for the device, and
            // the device may be running a kernel that waits for this very import.)
            if (s.pid == static_cast<int32_t>(getpid())) {
                // another rank of this very process: its address is valid here once peer access is on
                cudaError_t pe = cudaDeviceEnablePeerAccess(s.device, 0);
                if (pe == cudaSuccess || pe == cudaErrorPeerAccessAlreadyEnabled)
                    mapped = s.base;
            } else {
                void* base = nullptr;
                if (cudaIpcOpenMemHandle(&base, s.handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess) {
                    mapped = reinterpret_cast<uint64_t>(base);
                    to_close = base;
                } else {
                    MEGRAY_WARN("rank %u: could not map allocation %u of rank %u (%llu bytes)", m_rank, e, q,
                                static_cast<unsigned long long>(s.size));
                }
            }
            (void)cudaGetLastError();
            m_mappings[q].resize(e + 1, nullptr);
            m_mappings[q][e] = to_close;
            cudaMemcpyAsync(m_table_dev + static_cast<size_t>(q) * kMaxExports + e, &mapped, sizeof(mapped),
                            cudaMemcpyHostToDevice, m_stream);
            cudaStreamSynchronize(m_stream);
            (void)cudaGetLastError();
            ++m_imported[q];
            log(m_rank)->imported_from[q].store(m_imported[q], std::memory_order_release);
            m_imports_done.fetch_add(1);
            any = true;
        }
    }
    return any;
}

void IpcCache::helper_main() {
    cudaSetDevice(m_device);
    // Polls the peers' logs: every 50 us for a while after anything happened here or there (a new
    // buffer on one rank usually means new buffers on all), every millisecond otherwise.
    int busy_rounds = 0;
    while (!m_stop.load()) {
        if (import_new())
            busy_rounds = 400;
        std::unique_lock<std::mutex> lk(m_mu);
        if (m_kick) {
            m_kick = false;
            busy_rounds = 400;
            continue;
        }
        const auto nap = busy_rounds > 0 ? std::chrono::microseconds(50) : std::chrono::microseconds(1000);
        if (busy_rounds > 0)
            --busy_rounds;
        m_cv.wait_for(lk, nap, [this] { return m_kick; });
    }
}

}  // namespace MegRay
