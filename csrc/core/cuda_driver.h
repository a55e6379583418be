// Entry points of the CUDA driver API that the virtual-memory / multicast path
// needs, fetched at run time through the runtime (no link against libcuda, so
// the library also loads on a host without a GPU).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include "hccl/hccl_types.h"

namespace hccl {

struct DriverApi {
    CUresult (*cuMemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*cuMemRelease)(CUmemGenericAllocationHandle);
    CUresult (*cuMemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*cuMemAddressFree)(CUdeviceptr, size_t);
    CUresult (*cuMemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*cuMemUnmap)(CUdeviceptr, size_t);
    CUresult (*cuMemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*cuMemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*cuMemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType,
                                             unsigned long long);
    CUresult (*cuMemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
    CUresult (*cuMulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*cuMulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*cuMulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t,
                                   unsigned long long);
    CUresult (*cuMulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*cuMulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
    CUresult (*cuMemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr);
    CUresult (*cuDeviceGet)(CUdevice*, int);
    CUresult (*cuDeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*cuGetErrorString)(CUresult, const char**);
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    bool ok;
};

// nullptr when no driver is present (CPU-only host).
const DriverApi* GetDriverApi();
const char* DriverErrorString(CUresult r);

#define CHK_CU(expr)                                                                        \
    do {                                                                                    \
        CUresult _r = (expr);                                                               \
        if (_r != CUDA_SUCCESS) {                                                           \
            HCCL_ERROR("CUDA driver call failed: %s -> %s", #expr, ::hccl::DriverErrorString(_r)); \
            return HCCL_E_DRV;                                                              \
        }                                                                                   \
    } while (0)

}  // namespace hccl
