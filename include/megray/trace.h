/**
 * Operation tracing.  The reference has no tracing at all (no NVTX, no timers
 * outside its benchmark, test/performance.cpp:79-83).  Here every collective
 * call opens a TraceScope: an NVTX range named "megray::<op>" (visible to
 * NVIDIA's profilers) and, when tracing to a file is on (env MEGRAY_TRACE=path
 * or trace_enable), a host-side span that is written as Chrome-trace JSON
 * ("chrome://tracing" / Perfetto) by trace_dump or at process exit.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#include <string>

namespace MegRay {

/** Start collecting spans; they are written to `path` by trace_dump() and at exit. */
void trace_enable(const std::string& path);
void trace_disable();
bool trace_enabled();
/** Write the spans collected so far (all ranks of this process). Returns their number. */
size_t trace_dump();

class TraceScope {
public:
    TraceScope(const char* op, size_t bytes, uint32_t rank);
    ~TraceScope();
    TraceScope(const TraceScope&) = delete;
    TraceScope& operator=(const TraceScope&) = delete;

private:
    const char* m_op;
    size_t m_bytes;
    uint32_t m_rank;
    int64_t m_t0_us;
    bool m_file;
};

}  // namespace MegRay
