// Passing file descriptors between the processes of one machine: each rank
// binds an abstract-namespace Unix datagram socket named after the group and
// its rank; a descriptor travels as SCM_RIGHTS ancillary data together with the
// sender's rank.  Used to share cuMemCreate allocations (POSIX file-descriptor
// handles) between one-process-per-GPU ranks.
#pragma once
#include <stdint.h>

#include <string>

#include "megray/types.h"

namespace MegRay {

class FdChannel {
public:
    FdChannel() = default;
    ~FdChannel();
    FdChannel(const FdChannel&) = delete;
    FdChannel& operator=(const FdChannel&) = delete;

    /** Bind this rank's socket. `group` must be the same on all ranks and unique per group. */
    Status open(const std::string& group, uint32_t rank);
    /** Send descriptor `fd` (tagged with `tag`) to `peer`'s socket. */
    Status send_fd(uint32_t peer, int fd, uint32_t tag);
    /** Receive one descriptor; returns the sender's rank and tag. */
    Status recv_fd(int* fd, uint32_t* from, uint32_t* tag, int64_t timeout_ms);
    void close();

private:
    std::string m_group;
    uint32_t m_rank = 0;
    int m_sock = -1;
};

}  // namespace MegRay
