// Automatic registration of ordinary device buffers between ranks that are separate processes.
//
// The MegRay interface passes raw device pointers (include/megray/communicator.h:63-101 of the
// reference) and MegEngine runs one process per GPU, so a peer cannot address the buffer of a call
// until the allocation that holds it has been exported (cudaIpcGetMemHandle) and mapped on the
// peer's side (cudaIpcOpenMemHandle).  Doing that with a host exchange inside every call would
// make every call wait for every peer on the host.  Instead:
//
//   * a rank EXPORTS an allocation the first time one of its calls names a buffer inside it: the
//     handle goes into this rank's log in a shared-memory region (one log per rank, append only),
//     and from then on the rank identifies buffers of that allocation to its peers as
//     (entry number, offset) - which is what the single-pass kernels exchange in their first
//     barrier instead of addresses;
//   * a helper thread per rank IMPORTS whatever appears in the peers' logs and stores the mapped
//     base address into a table in device memory, indexed by (rank, entry number);
//   * the importer acknowledges in its own log, and a rank names an entry to its peers only once
//     every peer has acknowledged it; until then (a few calls) the buffer is replaced by one of two
//     bounce buffers that every peer mapped at init.  So no rank ever waits on the host for a
//     peer, and no kernel waits for a mapping (mapping was seen to stall for seconds while the
//     importing GPU is busy, which a waiting kernel would make worse).
//
// An allocation is recognised by its base address and CUDA buffer id: memory that was freed and
// allocated again at the same address gets a new entry (the old mapping stays open until the
// communicator goes: closing one waits for the device, which may be running a kernel that waits
// for an import).
// Memory that cannot be exported (virtual-memory-management allocations, host memory) is not
// handled here: the caller copies through a buffer of its own, which can.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <condition_variable>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include <cuda_runtime.h>

#include "host/shared_region.h"
#include "megray/client.h"
#include "megray/types.h"

namespace MegRay {

class IpcCache {
public:
    static constexpr uint32_t kMaxExports = 512;       // allocations one rank can export
    static constexpr uint64_t kImportFailed = 1;       // table value: the mapping could not be opened
    // what a rank publishes about a buffer: entry number in the high 16 bits, offset below
    static constexpr uint32_t kEntryNull = 0xFFFF;     // no buffer (rooted operations)
    static constexpr uint32_t kEntryHeap = 0xFFFE;     // offset into the rank's symmetric heap
    static uint64_t encode(uint32_t entry, uint64_t offset) { return (static_cast<uint64_t>(entry) << 48) | offset; }

    IpcCache() = default;
    ~IpcCache();
    IpcCache(const IpcCache&) = delete;
    IpcCache& operator=(const IpcCache&) = delete;

    /** Collective over the group: sets up the shared logs, the device table and the helper thread.
     *  Returns false (on every rank alike) when some rank could not, in which case nothing runs. */
    bool init(Client& client, uint32_t nranks, uint32_t rank, int device);

    /** The (entry, offset) of [p, p + bytes) for the peers, exporting its allocation if this is the
     *  first time.  False: the memory cannot be exported, the log is full, or the allocation is
     *  larger than auto_max_bytes() and `any_size` is false (such allocations are only exported
     *  through registration, which waits for the peers: mapping a large allocation was seen to
     *  wait for the importing device, which may be running a kernel that waits for the mapping). */
    bool resolve(const void* p, size_t bytes, uint64_t* word, bool any_size = false);

    /** The (entry, offset) of [p, p + bytes) if its allocation is exported AND every peer has
     *  acknowledged mapping it.  Otherwise false, after starting the export when that is possible
     *  (allocation up to auto_max_bytes()): the caller uses a bounce buffer for this call, and a
     *  later call finds the allocation mapped.  Never waits. */
    bool resolve_mapped(const void* p, size_t bytes, uint64_t* word);

    /** This rank's two bounce buffers (input, output side), mapped by every peer since init. */
    void* bounce(int which) const { return m_bounce[which]; }
    size_t bounce_bytes() const { return m_bounce_bytes; }

    /** True when [p, p + bytes) lies in an allocation that is exported and mapped by every peer. */
    bool mapped_everywhere(const void* p, size_t bytes);

    /** Exports the allocation of [p, p + bytes) whatever its size and waits until every peer has
     *  mapped it.  Collective by contract: every rank registers its corresponding buffer, at a
     *  point where no collective on it is in flight. */
    Status register_range(const void* p, size_t bytes, int64_t timeout_ms);

    size_t auto_max_bytes() const { return m_auto_max; }

    /** Device table: [rank q][entry e] -> where export e of rank q is mapped here (0: not yet). */
    const uint64_t* table() const { return m_table_dev; }

    uint32_t exports() const { return m_exports_made; }
    uint32_t imports() const { return m_imports_done.load(); }

private:
    struct ExportSlot {
        uint64_t buffer_id;
        uint64_t base;
        uint64_t size;
        int32_t pid;
        int32_t device;
        uint32_t supersedes;  // entry of the same rank that this one replaces (same base address), or ~0u
        uint32_t pad;
        cudaIpcMemHandle_t handle;
    };
    struct RankLog {
        std::atomic<uint32_t> count;
        uint32_t pad[15];
        // written by this log's rank as an importer: how many entries of rank q's log it has mapped
        std::atomic<uint32_t> imported_from[16];
        ExportSlot slots[kMaxExports];
    };
    RankLog* log(uint32_t q) { return reinterpret_cast<RankLog*>(m_region->slot(q)); }
    void helper_main();
    bool import_new();  // true if something was imported

    std::shared_ptr<host::SharedRegion> m_region;
    uint32_t m_nranks = 0, m_rank = 0;
    int m_device = 0;
    uint64_t* m_table_dev = nullptr;
    cudaStream_t m_stream = nullptr;  // the helper thread's
    std::thread m_helper;
    std::atomic<bool> m_stop{false};
    std::atomic<uint32_t> m_imports_done{0};
    std::mutex m_mu;
    std::mutex m_import_mu;  // import_new() runs on the helper thread and, before a launch, on the caller's
    size_t m_auto_max = 64u << 20;  // MEGRAY_IPC_AUTO_MAX_MB
    bool entry_acked(uint32_t entry);
    void* m_bounce[2] = {nullptr, nullptr};  // exported and mapped by every peer at init
    size_t m_bounce_bytes = 0;
    std::condition_variable m_cv;
    bool m_kick = false;
    // exporter side (calling thread)
    struct Known {
        uint64_t buffer_id;
        uint64_t size;
        uint32_t entry;
    };
    std::map<uint64_t, Known> m_known;  // allocation base -> its latest export
    uint32_t m_exports_made = 0;
    // importer side (helper thread)
    std::vector<uint32_t> m_imported;            // per rank: log entries processed
    std::vector<std::vector<void*>> m_mappings;  // per rank, per entry: mapping to close (or null)
};

}  // namespace MegRay
