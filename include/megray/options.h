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
