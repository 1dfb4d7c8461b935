// Environment-backed options (see include/megray/options.h for the variables).
#include "megray/options.h"

#include <stdlib.h>

#include <mutex>

#include "megray/debug.h"

namespace MegRay {

namespace {
int64_t env_i64(const char* name, int64_t dflt) {
    const char* e = getenv(name);
    if (e == nullptr || *e == 0)
        return dflt;
    char* end = nullptr;
    long long v = strtoll(e, &end, 10);
    return end == e ? dflt : static_cast<int64_t>(v);
}
std::string env_str(const char* name, const char* dflt) {
    const char* e = getenv(name);
    return std::string(e != nullptr ? e : dflt);
}
}  // namespace

Options Options::from_env() {
    Options o;
    o.log_level = MegRay::log_level();
    o.net_device = env_str("MEGRAY_NET_DEVICE", "");
    o.timeout_ms = env_i64("MEGRAY_TIMEOUT_MS", 600000);
    o.connect_timeout_ms = env_i64("MEGRAY_CONNECT_TIMEOUT_MS", 120000);
    o.device_timeout_ms = env_i64("MEGRAY_DEVICE_TIMEOUT_MS", 10000);
    o.heap_mb = env_i64("MEGRAY_HEAP_MB", 1024);
    o.algo = env_str("MEGRAY_ALGO", "auto");
    o.nvls = env_i64("MEGRAY_NVLS", 0) != 0;
    o.tune_file = env_str("MEGRAY_TUNE_FILE", "");
    o.trace_path = env_str("MEGRAY_TRACE", "");
    o.max_ctas = static_cast<int>(env_i64("MEGRAY_MAX_CTAS", 0));
    return o;
}

Options& global_options() {
    static Options opts = Options::from_env();
    return opts;
}

}  // namespace MegRay
