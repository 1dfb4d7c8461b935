// The few CUDA driver-API entry points the NVLink backend needs (virtual memory
// management and multicast objects), resolved at run time through
// cudaGetDriverEntryPoint so that the library has no link-time dependency on
// libcuda and still loads on a machine without a GPU driver.
#pragma once
#include <cuda.h>

namespace MegRay {
namespace drv {

struct Api {
    CUresult (*GetErrorString)(CUresult, const char**);
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*,
                                            CUmemAllocationGranularity_flags);
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*,
                          unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle,
                       unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle,
                                           CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*,
                                             CUmemAllocationHandleType);
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
    CUresult (*PointerGetAttributes)(unsigned int, CUpointer_attribute*, void**, CUdeviceptr);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle,
                                 size_t, size_t, unsigned long long);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*,
                                        CUmulticastGranularity_flags);
};

/** Resolved entry points, or nullptr when no CUDA driver is present. */
const Api* api();

/** Text for a CUresult (never null). */
const char* error_string(CUresult r);

}  // namespace drv
}  // namespace MegRay
