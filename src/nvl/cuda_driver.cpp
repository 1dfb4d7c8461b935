#include "nvl/cuda_driver.h"

#include <cuda_runtime_api.h>

#include <mutex>

#include "megray/debug.h"

namespace MegRay {
namespace drv {

namespace {
Api g_api;
bool g_ok = false;

template <typename F>
bool resolve(const char* name, F& out, bool required = true) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || f == nullptr) {
        (void)cudaGetLastError();
        out = nullptr;
        if (required)
            MEGRAY_DEBUG("driver entry point %s not available", name);
        return !required;
    }
    out = reinterpret_cast<F>(f);
    return true;
}
}  // namespace

const Api* api() {
    static std::once_flag once;
    std::call_once(once, [] {
        bool ok = true;
        ok &= resolve("cuGetErrorString", g_api.GetErrorString);
        ok &= resolve("cuMemGetAllocationGranularity", g_api.MemGetAllocationGranularity);
        ok &= resolve("cuMemCreate", g_api.MemCreate);
        ok &= resolve("cuMemRelease", g_api.MemRelease);
        ok &= resolve("cuMemAddressReserve", g_api.MemAddressReserve);
        ok &= resolve("cuMemAddressFree", g_api.MemAddressFree);
        ok &= resolve("cuMemMap", g_api.MemMap);
        ok &= resolve("cuMemUnmap", g_api.MemUnmap);
        ok &= resolve("cuMemSetAccess", g_api.MemSetAccess);
        ok &= resolve("cuMemExportToShareableHandle", g_api.MemExportToShareableHandle);
        ok &= resolve("cuMemImportFromShareableHandle", g_api.MemImportFromShareableHandle);
        ok &= resolve("cuDeviceGetAttribute", g_api.DeviceGetAttribute);
        ok &= resolve("cuMemGetAddressRange", g_api.MemGetAddressRange);
        ok &= resolve("cuPointerGetAttributes", g_api.PointerGetAttributes);
        resolve("cuMulticastCreate", g_api.MulticastCreate, false);
        resolve("cuMulticastAddDevice", g_api.MulticastAddDevice, false);
        resolve("cuMulticastBindMem", g_api.MulticastBindMem, false);
        resolve("cuMulticastUnbind", g_api.MulticastUnbind, false);
        resolve("cuMulticastGetGranularity", g_api.MulticastGetGranularity, false);
        g_ok = ok;
    });
    return g_ok ? &g_api : nullptr;
}

const char* error_string(CUresult r) {
    const Api* a = api();
    const char* s = nullptr;
    if (a != nullptr && a->GetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr)
        return s;
    return "unknown driver error";
}

}  // namespace drv
}  // namespace MegRay
