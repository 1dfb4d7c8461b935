// Symmetric heap: one cuMemCreate allocation per rank, mapped by every rank of
// the group, so that device code can load and store any peer's memory over
// NVLink.  Peers in the same process (thread-per-rank, as the reference's
// tests drive their ranks: test/test_base.h:46-51) share the allocation handle
// through a process-wide table; peers in other processes (one process per GPU)
// receive it as a POSIX file descriptor over a Unix socket.
//
// The reference has no peer-memory path of its own: all GPU-to-GPU bytes move
// inside NCCL/UCX or through host shared memory (src/shm/all_reduce.cpp:88-124).
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "megray/client.h"
#include "nvl/cuda_driver.h"

namespace MegRay {

class SymmetricHeap {
public:
    SymmetricHeap() = default;
    ~SymmetricHeap();
    SymmetricHeap(const SymmetricHeap&) = delete;
    SymmetricHeap& operator=(const SymmetricHeap&) = delete;

    /** Collective over the group behind `client`. The calling thread's current CUDA device is
     *  this rank's GPU. `group` is a string unique to this group on this machine. */
    Status create(Client* client, uint32_t nranks, uint32_t rank, size_t bytes,
                  const std::string& group, bool want_multicast);
    void destroy();

    size_t bytes() const { return m_bytes; }
    /** Rank q's heap as mapped in this rank's address space. */
    char* base(uint32_t q) const { return m_base[q]; }
    char* local() const { return m_base[m_rank]; }
    /** Multicast (NVSwitch) mapping of the heap: a store reaches all ranks, a multimem load
     *  reduces over all ranks.  nullptr when multicast is unavailable. */
    char* multicast() const { return m_mc_base; }
    int device() const { return m_device; }
    /** True when every rank of the group is a thread of this process (they then share one
     *  address space: a peer's device pointer means the same thing here). */
    bool same_process() const { return m_same_process; }
    /** CUDA device ordinal of rank q (meaningful for ranks of this process). */
    int peer_device(uint32_t q) const { return q < m_devices.size() ? m_devices[q] : -1; }

private:
    struct PeerInfo {
        int32_t pid;
        int32_t device;
        uint64_t host;
        uint64_t bytes;
        int32_t multicast_ok;
        int32_t pad;
    };
    Status exchange_handles(Client* client, const std::vector<PeerInfo>& info,
                            const std::string& group, CUmemGenericAllocationHandle mine,
                            std::vector<CUmemGenericAllocationHandle>* out, uint32_t tag);
    Status setup_multicast(Client* client, const std::vector<PeerInfo>& info,
                           const std::string& group);

    const drv::Api* m_api = nullptr;
    uint32_t m_nranks = 0, m_rank = 0;
    int m_device = -1;
    bool m_same_process = false;
    std::vector<int> m_devices;
    size_t m_bytes = 0;
    CUdeviceptr m_va = 0;
    std::vector<char*> m_base;
    std::vector<CUmemGenericAllocationHandle> m_handles;
    std::vector<bool> m_mapped;
    std::string m_group;
    CUmemGenericAllocationHandle m_mc_handle = 0;
    bool m_mc_bound = false;
    bool m_mc_owned = false;
    bool m_mc_shared = false;  // handle value shared with the other ranks of this process
    CUdeviceptr m_mc_va = 0;
    char* m_mc_base = nullptr;
};

}  // namespace MegRay
