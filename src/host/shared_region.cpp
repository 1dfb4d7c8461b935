#include "host/shared_region.h"

#include <errno.h>
#include <fcntl.h>
#include <sched.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <map>
#include <mutex>
#include <new>

#include "megray/debug.h"

namespace MegRay {
namespace host {

namespace {
constexpr uint32_t kMagic = 0x4d475259;  // "MGRY"
constexpr size_t kAlign = 4096;

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int64_t now_ms() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<int64_t>(ts.tv_sec) * 1000 + ts.tv_nsec / 1000000;
}

struct ProcEntry {
    void* base;
    size_t bytes;
    int refs;
};
std::mutex g_mu;
std::map<std::string, ProcEntry>& registry() {
    static std::map<std::string, ProcEntry> r;
    return r;
}
}  // namespace

size_t SharedRegion::total_bytes(uint32_t n, size_t slot, size_t mbox) {
    return round_up(sizeof(RegionHeader), kAlign) + (static_cast<size_t>(n) + 1) * slot +
           static_cast<size_t>(n) * n * (round_up(sizeof(Mailbox), 128) + mbox);
}

void SharedRegion::bind(void* base) {
    m_base = base;
    m_hdr = static_cast<RegionHeader*>(base);
    m_slots = static_cast<char*>(base) + round_up(sizeof(RegionHeader), kAlign);
    m_mail = m_slots + (static_cast<size_t>(m_hdr->nranks) + 1) * m_hdr->slot_bytes;
}

Mailbox* SharedRegion::mailbox(uint32_t from, uint32_t to) {
    size_t stride = round_up(sizeof(Mailbox), 128) + m_hdr->mailbox_bytes;
    return reinterpret_cast<Mailbox*>(m_mail + (static_cast<size_t>(from) * m_hdr->nranks + to) * stride);
}
char* SharedRegion::mailbox_data(uint32_t from, uint32_t to) {
    return reinterpret_cast<char*>(mailbox(from, to)) + round_up(sizeof(Mailbox), 128);
}

std::shared_ptr<SharedRegion> SharedRegion::create(const std::string& name, uint32_t nranks,
                                                   size_t slot_bytes, size_t mailbox_bytes,
                                                   bool in_process) {
    slot_bytes = round_up(slot_bytes, kAlign);
    mailbox_bytes = round_up(mailbox_bytes, kAlign);
    const size_t bytes = total_bytes(nranks, slot_bytes, mailbox_bytes);
    void* base = nullptr;
    if (in_process) {
        base = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_PRIVATE | MAP_ANONYMOUS, -1, 0);
        if (base == MAP_FAILED) {
            MEGRAY_ERROR("mmap %zu bytes: %s", bytes, strerror(errno));
            return nullptr;
        }
    } else {
        int fd = ::shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
        if (fd < 0) {
            MEGRAY_ERROR("shm_open(%s): %s", name.c_str(), strerror(errno));
            return nullptr;
        }
        if (::ftruncate(fd, static_cast<off_t>(bytes)) != 0) {
            MEGRAY_ERROR("ftruncate(%s, %zu): %s", name.c_str(), bytes, strerror(errno));
            ::close(fd);
            ::shm_unlink(name.c_str());
            return nullptr;
        }
        base = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
        ::close(fd);
        if (base == MAP_FAILED) {
            ::shm_unlink(name.c_str());
            return nullptr;
        }
    }
    // fresh mappings are zero-filled: atomics start at 0
    auto* hdr = new (base) RegionHeader;
    hdr->nranks = nranks;
    hdr->slot_bytes = slot_bytes;
    hdr->mailbox_bytes = mailbox_bytes;
    hdr->attached.store(1);
    hdr->aborted.store(0);
    hdr->barrier_count.store(0);
    hdr->barrier_sense.store(0);
    hdr->detached.store(0);
    std::atomic_thread_fence(std::memory_order_release);
    hdr->magic = kMagic;

    std::shared_ptr<SharedRegion> r(new SharedRegion);
    r->m_name = name;
    r->m_in_process = in_process;
    r->m_owner = true;
    r->m_bytes = bytes;
    r->bind(base);
    if (in_process) {
        std::lock_guard<std::mutex> lk(g_mu);
        registry()[name] = ProcEntry{base, bytes, 1};
    }
    return r;
}

std::shared_ptr<SharedRegion> SharedRegion::attach(const std::string& name, bool in_process,
                                                   int64_t timeout_ms) {
    const int64_t t0 = now_ms();
    void* base = nullptr;
    size_t bytes = 0;
    for (;;) {
        if (in_process) {
            std::lock_guard<std::mutex> lk(g_mu);
            auto it = registry().find(name);
            if (it != registry().end()) {
                base = it->second.base;
                bytes = it->second.bytes;
                it->second.refs++;
            }
        } else {
            int fd = ::shm_open(name.c_str(), O_RDWR, 0600);
            if (fd >= 0) {
                struct stat st;
                if (::fstat(fd, &st) == 0 && st.st_size >= static_cast<off_t>(sizeof(RegionHeader))) {
                    bytes = static_cast<size_t>(st.st_size);
                    base = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
                    if (base == MAP_FAILED)
                        base = nullptr;
                }
                ::close(fd);
            }
        }
        if (base != nullptr) {
            auto* hdr = static_cast<RegionHeader*>(base);
            // wait until the creator has finished the header
            while (reinterpret_cast<volatile uint32_t&>(hdr->magic) != kMagic) {
                if (timeout_ms > 0 && now_ms() - t0 > timeout_ms)
                    break;
                sched_yield();
            }
            std::atomic_thread_fence(std::memory_order_acquire);
            if (hdr->magic == kMagic)
                break;
        }
        if (timeout_ms > 0 && now_ms() - t0 > timeout_ms) {
            MEGRAY_ERROR("shared region %s did not appear within %lld ms", name.c_str(),
                         static_cast<long long>(timeout_ms));
            return nullptr;
        }
        usleep(200);
    }
    std::shared_ptr<SharedRegion> r(new SharedRegion);
    r->m_name = name;
    r->m_in_process = in_process;
    r->m_owner = false;
    r->m_bytes = bytes;
    r->bind(base);
    r->m_hdr->attached.fetch_add(1);
    return r;
}

SharedRegion::~SharedRegion() {
    if (m_base == nullptr)
        return;
    const uint32_t n = m_hdr->nranks;
    const uint32_t gone = m_hdr->detached.fetch_add(1) + 1;
    if (m_in_process) {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = registry().find(m_name);
        if (it != registry().end() && --it->second.refs == 0) {
            ::munmap(it->second.base, it->second.bytes);
            registry().erase(it);
        }
    } else {
        // the object's name is removed by whoever leaves last (or by the creator at the latest)
        if (gone >= n || m_owner)
            ::shm_unlink(m_name.c_str());
        ::munmap(m_base, m_bytes);
    }
}

Status SharedRegion::barrier(uint32_t* local_sense, int64_t timeout_ms) {
    RegionHeader* h = m_hdr;
    if (aborted())
        return MEGRAY_ABORTED;
    const uint32_t sense = *local_sense ^ 1u;
    *local_sense = sense;
    const uint32_t n = h->nranks;
    if (h->barrier_count.fetch_add(1, std::memory_order_acq_rel) + 1 == n) {
        h->barrier_count.store(0, std::memory_order_relaxed);
        h->barrier_sense.store(sense, std::memory_order_release);
        return MEGRAY_OK;
    }
    const int64_t t0 = now_ms();
    uint32_t spins = 0;
    while (h->barrier_sense.load(std::memory_order_acquire) != sense) {
        if (++spins < 2000)
            continue;
        sched_yield();
        if ((spins & 0x3ff) == 0) {
            if (aborted())
                return MEGRAY_ABORTED;
            if (timeout_ms > 0 && now_ms() - t0 > timeout_ms) {
                abort();  // the group cannot continue consistently after a missed barrier
                return MEGRAY_TIMEOUT;
            }
        }
    }
    return MEGRAY_OK;
}

}  // namespace host
}  // namespace MegRay
