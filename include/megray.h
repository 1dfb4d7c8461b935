/**
 * megray.h -- umbrella header of the B200-native MegRay-compatible collective library.
 *
 * Same entry points as the reference's include/megray.h:33-34
 * (`MegRay::get_communicator(nranks, rank, backend)`), plus the lower-case
 * namespace alias `megray`, the RAII `Server`, a host context and the native
 * NVLink backend selector `MEGRAY_NVL`.
 */
#pragma once

#include "megray/common.h"
#include "megray/communicator.h"
#include "megray/context.h"
#include "megray/options.h"
#include "megray/server.h"

#ifdef MEGRAY_WITH_CUDA
#include "megray/cuda_context.h"
#include "megray/fused.h"
#endif

#ifdef MEGRAY_WITH_HIP
#include "megray/hip_context.h"
#endif

namespace MegRay {

/**
 * Build a communicator for rank `rank` of `nranks`.
 *
 *   MEGRAY_NCCL  thin wrapper over NCCL (the baseline the native backend is measured against)
 *   MEGRAY_NVL   native sm_100a kernels over NVLink/NVSwitch peer memory (the product)
 *   MEGRAY_SHM   host backend: CPU ranks (threads or processes on one machine)
 *   MEGRAY_UCX / MEGRAY_RCCL  not built on this platform: throws MegRay::Exception
 *                ("unknown backend"), as a default build of the reference does
 *                (reference src/megray.cpp:56-57)
 */
std::shared_ptr<Communicator> get_communicator(uint32_t nranks, uint32_t rank, Backend backend);

}  // namespace MegRay

namespace megray = MegRay;
