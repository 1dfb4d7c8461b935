#include "nccl/nccl_loader.h"

#include <dlfcn.h>

#include <mutex>

#include "megray/debug.h"

namespace MegRay {
namespace nccl {

namespace {
Api g_api;
bool g_ok = false;

template <typename F>
bool sym(void* h, const char* name, F& out) {
    out = reinterpret_cast<F>(dlsym(h, name));
    if (out == nullptr)
        MEGRAY_ERROR("libnccl: missing symbol %s", name);
    return out != nullptr;
}
}  // namespace

const Api* api() {
    static std::once_flag once;
    std::call_once(once, [] {
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr)
            h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) {
            MEGRAY_WARN("cannot open libnccl.so.2: %s", dlerror());
            return;
        }
        bool ok = true;
        ok &= sym(h, "ncclGetVersion", g_api.GetVersion);
        ok &= sym(h, "ncclGetUniqueId", g_api.GetUniqueId);
        ok &= sym(h, "ncclCommInitRank", g_api.CommInitRank);
        ok &= sym(h, "ncclCommDestroy", g_api.CommDestroy);
        ok &= sym(h, "ncclCommAbort", g_api.CommAbort);
        ok &= sym(h, "ncclCommGetAsyncError", g_api.CommGetAsyncError);
        ok &= sym(h, "ncclGetErrorString", g_api.GetErrorString);
        ok &= sym(h, "ncclSend", g_api.Send);
        ok &= sym(h, "ncclRecv", g_api.Recv);
        ok &= sym(h, "ncclAllReduce", g_api.AllReduce);
        ok &= sym(h, "ncclAllGather", g_api.AllGather);
        ok &= sym(h, "ncclReduceScatter", g_api.ReduceScatter);
        ok &= sym(h, "ncclBroadcast", g_api.Broadcast);
        ok &= sym(h, "ncclReduce", g_api.Reduce);
        ok &= sym(h, "ncclGroupStart", g_api.GroupStart);
        ok &= sym(h, "ncclGroupEnd", g_api.GroupEnd);
        g_ok = ok;
    });
    return g_ok ? &g_api : nullptr;
}

}  // namespace nccl
}  // namespace MegRay
