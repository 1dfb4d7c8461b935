// Logger: one line per message on stderr,
//   [LEVEL] hh:mm:ss.mmm pid=<pid> rank=<r> file:line, message
// The reference prints "[LEVEL]\tfile:line, msg" with no time, pid or rank
// (src/core/debug.cpp:19-27).  The threshold starts at the compile-time
// MEGRAY_LOG_LEVEL and can be changed by env MEGRAY_LOG_LEVEL or set_log_level.
#include <stdarg.h>
#include <stdlib.h>
#include <string.h>
#include <sys/time.h>
#include <time.h>
#include <unistd.h>

#include <atomic>

#include "megray/debug.h"

namespace MegRay {

namespace {
std::atomic<int> g_level{-1};
thread_local int t_rank = -1;

int initial_level() {
    const char* e = getenv("MEGRAY_LOG_LEVEL");
    if (e != nullptr && *e != 0) {
        char* end = nullptr;
        long v = strtol(e, &end, 10);
        if (end != e && v >= 0 && v <= 3)
            return static_cast<int>(v);
        if (!strcasecmp(e, "debug")) return DEBUG;
        if (!strcasecmp(e, "info")) return INFO;
        if (!strcasecmp(e, "warn")) return WARN;
        if (!strcasecmp(e, "error")) return ERROR;
    }
    return MEGRAY_LOG_LEVEL;
}
}  // namespace

int log_level() {
    int l = g_level.load(std::memory_order_relaxed);
    if (l < 0) {
        l = initial_level();
        g_level.store(l, std::memory_order_relaxed);
    }
    return l;
}

void set_log_level(int level) {
    if (level < 0) level = 0;
    if (level > 3) level = 3;
    g_level.store(level, std::memory_order_relaxed);
}

void set_log_rank(int rank) { t_rank = rank; }

void MEGRAY_LOG(const char* level, const char* file, int line, const char* fmt, ...) {
    char msg[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(msg, sizeof(msg), fmt, ap);
    va_end(ap);
    struct timeval tv;
    gettimeofday(&tv, nullptr);
    struct tm tmv;
    localtime_r(&tv.tv_sec, &tmv);
    const char* base = strrchr(file, '/');
    base = base ? base + 1 : file;
    // one fprintf so that lines of concurrent ranks do not interleave
    fprintf(stderr, "[%s] %02d:%02d:%02d.%03d pid=%d rank=%d %s:%d, %s\n", level, tmv.tm_hour,
            tmv.tm_min, tmv.tm_sec, static_cast<int>(tv.tv_usec / 1000), static_cast<int>(getpid()),
            t_rank, base, line, msg);
}

}  // namespace MegRay
