// get_communicator: maps a Backend value to its implementation
// (reference src/megray.cpp:32-60).  Backends that are not part of this build
// throw "unknown backend", exactly like a reference build without them.
#include "megray.h"

#ifdef MEGRAY_WITH_SHM
#include "host/host_communicator.h"
#endif
#ifdef MEGRAY_WITH_NCCL
#include "nccl/nccl_communicator.h"
#endif
#ifdef MEGRAY_WITH_NVL
#include "nvl/nvl_communicator.h"
#endif

namespace MegRay {

std::shared_ptr<Communicator> get_communicator(uint32_t nranks, uint32_t rank, Backend backend) {
    if (nranks == 0 || rank >= nranks)
        MEGRAY_THROW("get_communicator: rank out of range");
    switch (backend) {
#ifdef MEGRAY_WITH_NCCL
        case MEGRAY_NCCL:
            return std::make_shared<NcclCommunicator>(nranks, rank);
#endif
#ifdef MEGRAY_WITH_NVL
        case MEGRAY_NVL:
            return std::make_shared<NvlCommunicator>(nranks, rank);
#endif
#ifdef MEGRAY_WITH_SHM
        case MEGRAY_SHM:
            return std::make_shared<HostCommunicator>(nranks, rank);
#endif
        default:
            // MEGRAY_UCX and MEGRAY_RCCL have no implementation on this platform.
            MEGRAY_THROW("unknown backend");
    }
}

}  // namespace MegRay
