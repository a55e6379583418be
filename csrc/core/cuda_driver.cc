#include "cuda_driver.h"
#include <mutex>
#include "log.h"

namespace hccl {
namespace {
DriverApi g_api;
std::once_flag g_once;

template <class F>
bool Load(const char* name, F* out)
{
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return false;
    }
    *out = reinterpret_cast<F>(fn);
    return true;
}
}  // namespace

const DriverApi* GetDriverApi()
{
    std::call_once(g_once, [] {
        g_api.ok = false;
        int n = 0;
        if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) { cudaGetLastError(); return; }
        bool ok = true;
#define L(name) ok = Load(#name, &g_api.name) && ok
        L(cuMemCreate); L(cuMemRelease); L(cuMemAddressReserve); L(cuMemAddressFree); L(cuMemMap); L(cuMemUnmap);
        L(cuMemSetAccess); L(cuMemGetAllocationGranularity); L(cuMemExportToShareableHandle);
        L(cuMemImportFromShareableHandle); L(cuDeviceGet); L(cuDeviceGetAttribute); L(cuGetErrorString);
        L(cuTensorMapEncodeTiled); L(cuMemGetAddressRange);
#undef L
        // multicast entry points are optional (older drivers): their absence only disables NVLS
        bool mc = true;
#define M(name) mc = Load(#name, &g_api.name) && mc
        M(cuMulticastCreate); M(cuMulticastAddDevice); M(cuMulticastBindMem); M(cuMulticastUnbind);
        M(cuMulticastGetGranularity);
#undef M
        if (!mc) g_api.cuMulticastCreate = nullptr;
        g_api.ok = ok;
    });
    return g_api.ok ? &g_api : nullptr;
}

const char* DriverErrorString(CUresult r)
{
    const DriverApi* d = GetDriverApi();
    const char* s = nullptr;
    if (d && d->cuGetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
    return "unknown driver error";
}

}  // namespace hccl
