// The memory that CPU ranks of one group share, and the synchronisation built
// in it: a sense-reversing barrier, per-rank staging slots, one result slot and
// a ring mailbox per ordered pair of ranks.
//
// Ranks that live in one process (threads, as the reference's tests run them:
// test/test_base.h:46-51) share a heap block found through a process-wide
// registry; ranks in different processes map a POSIX shared-memory object.
// The reference's host backend uses a SysV segment plus per-message POSIX
// objects and synchronises through plain `volatile int` words
// (src/shm/communicator.cpp:156-188, src/shm/shm_barrier.cpp:16-47); here every
// shared word is a std::atomic and every wait has a deadline.
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <atomic>
#include <memory>
#include <string>

#include "megray/types.h"

namespace MegRay {
namespace host {

struct RegionHeader {
    uint32_t magic;
    uint32_t nranks;
    uint64_t slot_bytes;
    uint64_t mailbox_bytes;
    std::atomic<uint32_t> attached;  // ranks that have mapped the region
    std::atomic<uint32_t> aborted;   // set by a rank whose wait ran out or that was aborted
    std::atomic<uint32_t> barrier_count;
    std::atomic<uint32_t> barrier_sense;
    std::atomic<uint32_t> detached;
};

struct Mailbox {
    std::atomic<uint64_t> head;  // bytes written so far (sender)
    char pad0[56];
    std::atomic<uint64_t> tail;  // bytes read so far (receiver)
    char pad1[56];
    // followed by mailbox_bytes of ring storage
};

class SharedRegion {
public:
    /** Geometry is fixed by rank 0; `name` identifies the group on this machine. */
    static std::shared_ptr<SharedRegion> create(const std::string& name, uint32_t nranks,
                                                size_t slot_bytes, size_t mailbox_bytes,
                                                bool in_process);
    /** Attach to a region created by rank 0 (waits for it to appear, up to timeout_ms). */
    static std::shared_ptr<SharedRegion> attach(const std::string& name, bool in_process,
                                                int64_t timeout_ms);
    ~SharedRegion();

    RegionHeader* header() { return m_hdr; }
    uint32_t nranks() const { return m_hdr->nranks; }
    size_t slot_bytes() const { return m_hdr->slot_bytes; }
    size_t mailbox_bytes() const { return m_hdr->mailbox_bytes; }
    char* slot(uint32_t rank) { return m_slots + static_cast<size_t>(rank) * m_hdr->slot_bytes; }
    char* result() { return m_slots + static_cast<size_t>(m_hdr->nranks) * m_hdr->slot_bytes; }
    Mailbox* mailbox(uint32_t from, uint32_t to);
    char* mailbox_data(uint32_t from, uint32_t to);

    /** All ranks meet; MEGRAY_TIMEOUT after timeout_ms, MEGRAY_ABORTED if the group was aborted.
     *  `local_sense` is the caller's private sense word (starts at 0). */
    Status barrier(uint32_t* local_sense, int64_t timeout_ms);

    void abort() { m_hdr->aborted.store(1, std::memory_order_release); }
    bool aborted() const { return m_hdr->aborted.load(std::memory_order_acquire) != 0; }

private:
    SharedRegion() = default;
    static size_t total_bytes(uint32_t nranks, size_t slot_bytes, size_t mailbox_bytes);
    void bind(void* base);

    std::string m_name;
    bool m_in_process = false;
    bool m_owner = false;
    void* m_base = nullptr;
    size_t m_bytes = 0;
    RegionHeader* m_hdr = nullptr;
    char* m_slots = nullptr;
    char* m_mail = nullptr;
};

}  // namespace host
}  // namespace MegRay
