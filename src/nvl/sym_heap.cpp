#include "nvl/sym_heap.h"

#include <cuda_runtime_api.h>
#include <string.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <map>
#include <mutex>

#include "megray/common.h"
#include "megray/options.h"
#include "nvl/fd_channel.h"

namespace MegRay {

namespace {

#define DRV_CHECK(expr)                                                                 \
    do {                                                                                \
        CUresult megray_cu_ = (expr);                                                   \
        if (megray_cu_ != CUDA_SUCCESS) {                                               \
            MEGRAY_ERROR("driver error [%d] %s in %s", megray_cu_,                      \
                         drv::error_string(megray_cu_), #expr);                         \
            return MEGRAY_CUDA_ERR;                                                     \
        }                                                                               \
    } while (0)

// Handles published by ranks of this process, keyed by "<group>:<tag>:<rank>".
struct HandleTable {
    std::mutex mu;
    std::condition_variable cv;
    std::map<std::string, CUmemGenericAllocationHandle> map;
    // multicast objects used by several ranks of this process through one handle value: the
    // last user to let go releases the object
    std::map<CUmemGenericAllocationHandle, int> mc_users;
};
HandleTable& table() {
    static HandleTable t;
    return t;
}
std::string key_of(const std::string& group, uint32_t tag, uint32_t rank) {
    return group + ":" + std::to_string(tag) + ":" + std::to_string(rank);
}

uint64_t host_hash() {
    char name[256] = {0};
    gethostname(name, sizeof(name) - 1);
    uint64_t h = 1469598103934665603ull;
    for (const char* p = name; *p; ++p)
        h = (h ^ static_cast<unsigned char>(*p)) * 1099511628211ull;
    // the boot id tells apart containers that share a host name
    return h;
}

CUmemAllocationProp heap_prop(int device) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

}  // namespace

SymmetricHeap::~SymmetricHeap() { destroy(); }

void SymmetricHeap::destroy() {
    if (m_api == nullptr)
        return;
    if (m_device >= 0)
        cudaSetDevice(m_device);
    if (m_mc_base != nullptr) {
        m_api->MemUnmap(m_mc_va, m_bytes);
        m_api->MemAddressFree(m_mc_va, m_bytes);
        m_mc_base = nullptr;
    }
    if (m_mc_handle != 0) {
        if (m_mc_bound && m_api->MulticastUnbind != nullptr)
            m_api->MulticastUnbind(m_mc_handle, m_device, 0, m_bytes);
        bool release = m_mc_owned;
        if (m_mc_shared) {
            // the handle value is shared with the other ranks of this process, which may still
            // be unbinding: only the last one releases it
            HandleTable& t = table();
            std::lock_guard<std::mutex> lk(t.mu);
            auto it = t.mc_users.find(m_mc_handle);
            release = it != t.mc_users.end() && --it->second == 0;
            if (release)
                t.mc_users.erase(it);
        }
        if (release)
            m_api->MemRelease(m_mc_handle);
        m_mc_handle = 0;
        m_mc_shared = false;
    }
    for (uint32_t q = 0; q < m_base.size(); ++q) {
        if (m_mapped.size() > q && m_mapped[q])
            m_api->MemUnmap(m_va + static_cast<size_t>(q) * m_bytes, m_bytes);
    }
    for (uint32_t q = 0; q < m_handles.size(); ++q)
        if (m_handles[q] != 0)
            m_api->MemRelease(m_handles[q]);
    if (m_va != 0)
        m_api->MemAddressFree(m_va, m_bytes * m_nranks);
    {
        HandleTable& t = table();
        std::lock_guard<std::mutex> lk(t.mu);
        for (uint32_t tag = 0; tag < 2; ++tag)
            t.map.erase(key_of(m_group, tag, m_rank));
    }
    m_handles.clear();
    m_base.clear();
    m_mapped.clear();
    m_va = 0;
    m_api = nullptr;
}

Status SymmetricHeap::exchange_handles(Client* client, const std::vector<PeerInfo>& info,
                                       const std::string& group, CUmemGenericAllocationHandle mine,
                                       std::vector<CUmemGenericAllocationHandle>* out,
                                       uint32_t tag) {
    const uint32_t n = m_nranks;
    out->assign(n, 0);
    (*out)[m_rank] = mine;
    const int32_t my_pid = info[m_rank].pid;
    uint32_t remote = 0;
    for (uint32_t q = 0; q < n; ++q)
        if (q != m_rank && info[q].pid != my_pid)
            ++remote;

    // same-process peers: through the table
    {
        HandleTable& t = table();
        std::unique_lock<std::mutex> lk(t.mu);
        t.map[key_of(group, tag, m_rank)] = mine;
        t.cv.notify_all();
        const auto deadline = std::chrono::steady_clock::now() +
                              std::chrono::milliseconds(global_options().connect_timeout_ms);
        for (uint32_t q = 0; q < n; ++q) {
            if (q == m_rank || info[q].pid != my_pid)
                continue;
            const std::string k = key_of(group, tag, q);
            while (t.map.find(k) == t.map.end()) {
                if (t.cv.wait_until(lk, deadline) == std::cv_status::timeout) {
                    MEGRAY_ERROR("rank %u: peer %u never published its allocation", m_rank, q);
                    return MEGRAY_TIMEOUT;
                }
            }
            (*out)[q] = t.map[k];
        }
    }

    // other processes: POSIX file descriptors over a Unix socket
    FdChannel chan;
    int my_fd = -1;
    if (remote > 0) {
        MEGRAY_CHECK(chan.open(group + "-" + std::to_string(tag), m_rank));
        DRV_CHECK(m_api->MemExportToShareableHandle(&my_fd, mine,
                                                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    }
    MEGRAY_CHECK(client->barrier());  // every socket is bound
    if (remote > 0) {
        for (uint32_t q = 0; q < n; ++q)
            if (q != m_rank && info[q].pid != my_pid)
                MEGRAY_CHECK(chan.send_fd(q, my_fd, tag));
        for (uint32_t i = 0; i < remote; ++i) {
            int fd = -1;
            uint32_t from = 0, got_tag = 0;
            MEGRAY_CHECK(chan.recv_fd(&fd, &from, &got_tag, global_options().connect_timeout_ms));
            if (from >= n || got_tag != tag || (*out)[from] != 0) {
                ::close(fd);
                MEGRAY_ERROR("unexpected descriptor from rank %u", from);
                return MEGRAY_UNEXPECTED_ERR;
            }
            CUmemGenericAllocationHandle h = 0;
            CUresult r = m_api->MemImportFromShareableHandle(
                    &h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)),
                    CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            ::close(fd);
            if (r != CUDA_SUCCESS) {
                MEGRAY_ERROR("import of rank %u's allocation failed: %s", from, drv::error_string(r));
                return MEGRAY_CUDA_ERR;
            }
            (*out)[from] = h;
        }
        ::close(my_fd);
    }
    MEGRAY_CHECK(client->barrier());  // all descriptors delivered before the sockets close
    return MEGRAY_OK;
}

Status SymmetricHeap::create(Client* client, uint32_t nranks, uint32_t rank, size_t bytes,
                             const std::string& group, bool want_multicast) {
    m_api = drv::api();
    if (m_api == nullptr) {
        MEGRAY_ERROR("CUDA driver entry points are not available");
        return MEGRAY_ENV_ERROR;
    }
    m_nranks = nranks;
    m_rank = rank;
    m_group = group;
    CUDA_CHECK(cudaGetDevice(&m_device));
    CUDA_CHECK(cudaFree(nullptr));  // makes the primary context current on this thread

    CUmemAllocationProp prop = heap_prop(m_device);
    size_t gran = 0;
    DRV_CHECK(m_api->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    int mc_ok = 0;
    if (want_multicast && m_api->MulticastCreate != nullptr)
        m_api->DeviceGetAttribute(&mc_ok, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, m_device);
    if (mc_ok && nranks > 1) {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = nranks;
        mp.size = bytes;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        if (m_api->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) ==
                    CUDA_SUCCESS &&
            mg > gran)
            gran = mg;
    }
    bytes = (bytes + gran - 1) / gran * gran;

    std::vector<PeerInfo> info(nranks);
    PeerInfo me;
    memset(&me, 0, sizeof(me));
    me.pid = static_cast<int32_t>(getpid());
    me.device = m_device;
    me.host = host_hash();
    me.bytes = bytes;
    me.multicast_ok = mc_ok;
    MEGRAY_CHECK(client->allgather(&me, info.data(), sizeof(me)));
    bool all_mc = nranks > 1;
    for (uint32_t q = 0; q < nranks; ++q) {
        if (info[q].host != me.host) {
            MEGRAY_ERROR("NVL backend: rank %u is on another host; one NVSwitch domain only", q);
            return MEGRAY_INVALID_USAGE;
        }
        if (info[q].bytes != bytes) {
            MEGRAY_ERROR("NVL backend: rank %u asked for a %llu-byte heap, this rank for %zu", q,
                         static_cast<unsigned long long>(info[q].bytes), bytes);
            return MEGRAY_INVALID_USAGE;
        }
        if (q != rank && info[q].pid == me.pid && info[q].device == m_device) {
            MEGRAY_ERROR("NVL backend: ranks %u and %u share GPU %d", rank, q, m_device);
            return MEGRAY_INVALID_USAGE;
        }
        all_mc = all_mc && info[q].multicast_ok != 0;
    }
    m_bytes = bytes;
    m_same_process = true;
    m_devices.assign(nranks, -1);
    for (uint32_t q = 0; q < nranks; ++q) {
        m_devices[q] = info[q].device;
        if (info[q].pid != me.pid)
            m_same_process = false;
    }

    CUmemGenericAllocationHandle mine = 0;
    DRV_CHECK(m_api->MemCreate(&mine, bytes, &prop, 0));
    m_handles.assign(nranks, 0);
    m_handles[rank] = mine;
    DRV_CHECK(m_api->MemAddressReserve(&m_va, bytes * nranks, gran, 0, 0));
    m_base.assign(nranks, nullptr);
    m_mapped.assign(nranks, false);

    std::vector<CUmemGenericAllocationHandle> all;
    MEGRAY_CHECK(exchange_handles(client, info, group, mine, &all, 0));
    // handles of same-process peers are borrowed (their owner releases them); imported ones are ours
    for (uint32_t q = 0; q < nranks; ++q)
        if (q != rank && info[q].pid != me.pid)
            m_handles[q] = all[q];

    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = m_device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (uint32_t q = 0; q < nranks; ++q) {
        const CUdeviceptr at = m_va + static_cast<size_t>(q) * bytes;
        DRV_CHECK(m_api->MemMap(at, bytes, 0, all[q], 0));
        m_mapped[q] = true;
        DRV_CHECK(m_api->MemSetAccess(at, bytes, &acc, 1));
        m_base[q] = reinterpret_cast<char*>(at);
    }
    // flags and counters start at zero
    CUDA_CHECK(cudaMemset(m_base[rank], 0, bytes));
    CUDA_CHECK(cudaDeviceSynchronize());
    MEGRAY_CHECK(client->barrier());

    if (all_mc) {
        Status s = setup_multicast(client, info, group);
        if (s != MEGRAY_OK)
            MEGRAY_WARN("NVSwitch multicast not set up (status %d); using peer loads/stores only", s);
    }
    return MEGRAY_OK;
}

Status SymmetricHeap::setup_multicast(Client* client, const std::vector<PeerInfo>& info,
                                      const std::string& group) {
    // Rank 0 creates the multicast object; every rank adds its device, binds its heap
    // allocation at offset 0 and maps the object.  All ranks must take every collective
    // step (allgather/barrier) even after a local failure, so failures are voted on.
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = m_nranks;
    mp.size = m_bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    int32_t ok = 1;
    CUmemGenericAllocationHandle mc = 0;
    if (m_rank == 0 && m_api->MulticastCreate(&mc, &mp) != CUDA_SUCCESS)
        ok = 0;
    std::vector<int32_t> votes(m_nranks);
    MEGRAY_CHECK(client->allgather(&ok, votes.data(), sizeof(ok)));
    if (votes[0] == 0)
        return MEGRAY_NOT_IMPLEMENTED;

    // share rank 0's object: peers in this process through the table, others by descriptor
    const int32_t my_pid = info[m_rank].pid;
    std::vector<CUmemGenericAllocationHandle> all;
    if (m_rank == 0) {
        MEGRAY_CHECK(exchange_handles(client, info, group, mc, &all, 1));
    } else {
        // non-zero ranks publish nothing useful (their own heap handle) but take the same steps
        MEGRAY_CHECK(exchange_handles(client, info, group, m_handles[m_rank], &all, 1));
        mc = all[0];
        // imported copies of peers' heap handles (other than rank 0's object) are not needed
        for (uint32_t q = 1; q < m_nranks; ++q)
            if (q != m_rank && info[q].pid != my_pid && all[q] != 0)
                m_api->MemRelease(all[q]);
    }
    if (m_rank == 0)
        for (uint32_t q = 1; q < m_nranks; ++q)
            if (info[q].pid != my_pid && all[q] != 0)
                m_api->MemRelease(all[q]);
    const bool borrowed = m_rank != 0 && info[0].pid == my_pid;

    ok = m_api->MulticastAddDevice(mc, m_device) == CUDA_SUCCESS ? 1 : 0;
    MEGRAY_CHECK(client->allgather(&ok, votes.data(), sizeof(ok)));
    bool all_ok = true;
    for (int32_t v : votes)
        all_ok = all_ok && v != 0;
    if (all_ok) {
        ok = m_api->MulticastBindMem(mc, 0, m_handles[m_rank], 0, m_bytes, 0) == CUDA_SUCCESS ? 1 : 0;
        m_mc_bound = ok != 0;
        MEGRAY_CHECK(client->allgather(&ok, votes.data(), sizeof(ok)));
        for (int32_t v : votes)
            all_ok = all_ok && v != 0;
    }
    if (all_ok) {
        CUmemAccessDesc acc;
        memset(&acc, 0, sizeof(acc));
        acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        acc.location.id = m_device;
        acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
        CUdeviceptr va = 0;
        if (m_api->MemAddressReserve(&va, m_bytes, 0, 0, 0) == CUDA_SUCCESS) {
            if (m_api->MemMap(va, m_bytes, 0, mc, 0) == CUDA_SUCCESS &&
                m_api->MemSetAccess(va, m_bytes, &acc, 1) == CUDA_SUCCESS) {
                m_mc_va = va;
                m_mc_base = reinterpret_cast<char*>(va);
            } else {
                m_api->MemAddressFree(va, m_bytes);
            }
        }
        ok = m_mc_base != nullptr ? 1 : 0;
        MEGRAY_CHECK(client->allgather(&ok, votes.data(), sizeof(ok)));
        for (int32_t v : votes)
            all_ok = all_ok && v != 0;
    }
    m_mc_handle = mc;
    // rank 0's handle value serves every rank of rank 0's process (counted, the last user
    // releases it); ranks of other processes own the handle they imported
    m_mc_shared = info[0].pid == my_pid;
    m_mc_owned = !m_mc_shared;
    (void)borrowed;
    if (m_mc_shared) {
        HandleTable& t = table();
        std::lock_guard<std::mutex> lk(t.mu);
        t.mc_users[mc] += 1;
    }
    if (!all_ok) {
        if (m_mc_base != nullptr) {
            m_api->MemUnmap(m_mc_va, m_bytes);
            m_api->MemAddressFree(m_mc_va, m_bytes);
            m_mc_base = nullptr;
        }
        return MEGRAY_NOT_IMPLEMENTED;
    }
    return MEGRAY_OK;
}

}  // namespace MegRay
