/**
 * Run-time options, read once from the environment and overridable from code.
 * The reference has no such registry: its only run-time switches are
 * MEGRAY_NET_DEVICE (src/core/server.cpp:29) and NCCL_LAUNCH_MODE
 * (src/nccl/communicator.cpp:22).
 *
 *   MEGRAY_LOG_LEVEL    0..3            log threshold (default: compile-time level)
 *   MEGRAY_NET_DEVICE   iface name      interface whose address get_host_ip() returns
 *   MEGRAY_TIMEOUT_MS   milliseconds    limit of one rendezvous wait / host-backend wait
 *   MEGRAY_CONNECT_TIMEOUT_MS           limit for Client::connect (default 120 s)
 *   MEGRAY_DEVICE_TIMEOUT_MS            limit of one in-kernel flag wait (default 10 s)
 *   MEGRAY_HEAP_MB      MiB             symmetric heap per rank (default 1024)
 *   MEGRAY_ALGO         name            force an algorithm: oneshot | twoshot | nvls | auto
 *   MEGRAY_NVLS         0|1             allow NVSwitch multicast (multimem) paths
 *   MEGRAY_TUNE_FILE    path            JSON table of algorithm crossover points
 *   MEGRAY_TRACE        path            write a Chrome-trace JSON of every operation
 *   MEGRAY_MAX_CTAS     n               cap on CTAs of a collective kernel
 *
 * Read by the NVL backend itself when a communicator is created (tuning and diagnosis; the
 * tune table sets the same values, the environment overrides it):
 *   MEGRAY_TUNE_DEFAULT 0|1             load tune/tune_b200_n<ranks>.json beside the library (default 1)
 *   MEGRAY_LL_BYTES     bytes           flagged-word kernel up to this payload per pair of ranks (all operations)
 *   MEGRAY_ONESHOT_BYTES, MEGRAY_CTA_BYTES, MEGRAY_DIRECT_CTA_BYTES, MEGRAY_WORKSPACE_MB
 *                                       crossover of the one-shot all_reduce, bytes per CTA, staging size
 *   MEGRAY_DIRECT, MEGRAY_EXCHANGE, MEGRAY_PUSH_EXCHANGE   0 switches a kernel family / form off
 *   MEGRAY_IPC_CACHE    0|1             separate processes: export allocations on first use (default 1)
 *   MEGRAY_IPC_AUTO_MAX_MB              largest allocation exported without register_buffer (default 64)
 *   MEGRAY_BCAST_CHUNK  bytes           chunk of the pipelined broadcast and the staged reduces
 *   MEGRAY_BCAST_PULL, MEGRAY_BCAST_PULL_MIN   broadcast by loads alone, from this size on (default off)
 *   MEGRAY_REDUCE_MODE  0..3, MEGRAY_REDUCE_STAGED_MIN, MEGRAY_REDUCE_STEPS   form of a large reduce
 *   MEGRAY_SPIN_SLEEP_NS                pause between the polls of a wait that has lasted a while
 *   MEGRAY_NVL_P2P      0|1             set up the NCCL engine behind send / recv (default 1)
 *   MEGRAY_PHASES       0|1             kernels stamp %globaltimer at their phase boundaries
 */
#pragma once
#include <stdint.h>

#include <string>

namespace MegRay {

struct Options {
    int log_level;
    std::string net_device;
    int64_t timeout_ms;
    int64_t connect_timeout_ms;
    int64_t device_timeout_ms;
    int64_t heap_mb;
    std::string algo;
    bool nvls;
    std::string tune_file;
    std::string trace_path;
    int max_ctas;

    /** Options parsed from the environment (fresh parse on every call). */
    static Options from_env();
};

/** Process-wide options: first use parses the environment. */
Options& global_options();

}  // namespace MegRay
