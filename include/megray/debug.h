/**
 * Logging, exception type and assertion macros.
 *
 * Macro names and the printf-style calling convention follow the reference
 * (include/megray/debug.h:21-72).  Differences: the level can also be set at
 * run time (env MEGRAY_LOG_LEVEL=0..3 or set_log_level), and each line carries
 * a time stamp, the process id and, once known, the rank.
 */
#pragma once
#include <cstdio>
#include <stdexcept>
#include <string>

#include "megray/config.h"

namespace MegRay {

typedef enum { DEBUG = 0, INFO = 1, WARN = 2, ERROR = 3 } LogLevel;

/** Current threshold: messages below it are dropped. */
int log_level();
void set_log_level(int level);
/** Rank printed in the log prefix of the calling thread (-1 = unknown). */
void set_log_rank(int rank);

void MEGRAY_LOG(const char* level, const char* file, int line, const char* fmt, ...)
        __attribute__((format(printf, 4, 5)));

#define MEGRAY_LOG_AT(lvl, name, fmt...)                           \
    do {                                                           \
        if (static_cast<int>(lvl) >= MegRay::log_level()) {        \
            MegRay::MEGRAY_LOG(name, __FILE__, __LINE__, fmt);     \
        }                                                          \
    } while (0)

#define MEGRAY_DEBUG(fmt...) MEGRAY_LOG_AT(MegRay::LogLevel::DEBUG, "DEBUG", fmt)
#define MEGRAY_INFO(fmt...) MEGRAY_LOG_AT(MegRay::LogLevel::INFO, "INFO", fmt)
#define MEGRAY_WARN(fmt...) MEGRAY_LOG_AT(MegRay::LogLevel::WARN, "WARN", fmt)
#define MEGRAY_ERROR(fmt...) MEGRAY_LOG_AT(MegRay::LogLevel::ERROR, "ERROR", fmt)

class Exception : public std::runtime_error {
public:
    explicit Exception(const std::string& msg) : std::runtime_error(msg) {}
};

#define MEGRAY_THROW(message) throw MegRay::Exception(message)

#define MEGRAY_ASSERT(expr, fmt...)                      \
    do {                                                 \
        if (!(expr)) {                                   \
            MEGRAY_ERROR("assertion failed: %s", #expr); \
            MEGRAY_ERROR(fmt);                           \
            MEGRAY_THROW("assertion failed");            \
        }                                                \
    } while (0)

}  // namespace MegRay
