#include "megray/trace.h"

#include <stdio.h>
#include <stdlib.h>
#include <sys/syscall.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "megray/options.h"

#ifdef MEGRAY_WITH_CUDA
#include <nvtx3/nvToolsExt.h>
#endif

namespace MegRay {

namespace {
struct Span {
    const char* op;
    size_t bytes;
    uint32_t rank;
    int64_t t0_us, t1_us;
    long tid;
};
std::mutex g_mu;
std::vector<Span> g_spans;
std::string g_path;
std::atomic<int> g_state{-1};  // -1 unknown, 0 off, 1 on
constexpr size_t kMaxSpans = 1u << 20;

int64_t now_us() {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return static_cast<int64_t>(ts.tv_sec) * 1000000 + ts.tv_nsec / 1000;
}

void at_exit_dump() { trace_dump(); }

void init_from_env() {
    int expected = -1;
    const std::string& p = global_options().trace_path;
    if (g_state.compare_exchange_strong(expected, p.empty() ? 0 : 1) && !p.empty()) {
        std::lock_guard<std::mutex> lk(g_mu);
        g_path = p;
        atexit(at_exit_dump);
    }
}
}  // namespace

void trace_enable(const std::string& path) {
    bool first;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        first = g_path.empty();
        g_path = path;
    }
    g_state.store(1);
    if (first)
        atexit(at_exit_dump);
}

void trace_disable() { g_state.store(0); }

bool trace_enabled() {
    if (g_state.load(std::memory_order_relaxed) < 0)
        init_from_env();
    return g_state.load(std::memory_order_relaxed) == 1;
}

size_t trace_dump() {
    std::lock_guard<std::mutex> lk(g_mu);
    if (g_path.empty())
        return 0;
    std::string path = g_path;
    // one file per process when several processes share the setting
    const size_t pct = path.find("%p");
    if (pct != std::string::npos)
        path.replace(pct, 2, std::to_string(getpid()));
    FILE* f = fopen(path.c_str(), "w");
    if (f == nullptr)
        return 0;
    fprintf(f, "{\"traceEvents\":[\n");
    for (size_t i = 0; i < g_spans.size(); ++i) {
        const Span& s = g_spans[i];
        fprintf(f,
                "%s{\"name\":\"%s\",\"cat\":\"megray\",\"ph\":\"X\",\"ts\":%lld,\"dur\":%lld,"
                "\"pid\":%u,\"tid\":%ld,\"args\":{\"bytes\":%zu}}",
                i ? ",\n" : "", s.op, static_cast<long long>(s.t0_us),
                static_cast<long long>(s.t1_us - s.t0_us), s.rank, s.tid, s.bytes);
    }
    fprintf(f, "\n]}\n");
    fclose(f);
    return g_spans.size();
}

TraceScope::TraceScope(const char* op, size_t bytes, uint32_t rank)
        : m_op(op), m_bytes(bytes), m_rank(rank), m_t0_us(0), m_file(trace_enabled()) {
#ifdef MEGRAY_WITH_CUDA
    // NVTX binds its entry points on the first call, without synchronisation of its own: rank
    // threads that make their first call together would race there, so the first call is made
    // once, alone.
    static std::once_flag nvtx_bound;
    std::call_once(nvtx_bound, [] {
        nvtxRangePushA("megray::init");
        nvtxRangePop();
    });
    nvtxRangePushA(op);
#endif
    if (m_file)
        m_t0_us = now_us();
}

TraceScope::~TraceScope() {
#ifdef MEGRAY_WITH_CUDA
    nvtxRangePop();
#endif
    if (m_file) {
        Span s{m_op, m_bytes, m_rank, m_t0_us, now_us(), static_cast<long>(syscall(SYS_gettid))};
        std::lock_guard<std::mutex> lk(g_mu);
        if (g_spans.size() < kMaxSpans)
            g_spans.push_back(s);
    }
}

}  // namespace MegRay
