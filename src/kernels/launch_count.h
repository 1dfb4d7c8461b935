// Process-wide count of kernels launched by this library, so that a benchmark
// can report how many of the library's own kernels ran inside a timed region.
#pragma once
#include <atomic>
#include <stdint.h>

namespace mgk {
inline std::atomic<uint64_t>& launch_counter() {
    static std::atomic<uint64_t> c{0};
    return c;
}
inline void count_launch(uint64_t n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }
inline uint64_t launch_count() { return launch_counter().load(std::memory_order_relaxed); }
}  // namespace mgk
