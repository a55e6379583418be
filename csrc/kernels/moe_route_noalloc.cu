// HcclMoeExpertOffsetsNoAlloc: the expert-offsets kernel with its counters in a file-scope device array instead of
// a cudaMalloc'ed buffer, for callers that cannot allocate (see hccl/hccl_moe_noalloc.h for who they are and what
// the variant costs).  Nothing in this file allocates: no cudaMalloc / cudaFree, no containers that grow on the
// call path, no library routine that allocates device memory.
#include <cuda_runtime.h>
#include "../core/log.h"
#include "hccl/hccl_moe_noalloc.h"
#include "moe_route.cuh"

namespace {

// Counters [0, max) and the exit ticket [max].  Zero-initialised by the loader; the kernel restores the zeros
// before it ends.  Every device that loads this module owns one copy for the lifetime of the process.
static __device__ __align__(256) uint32_t g_routeScratch[HCCL_MOE_NOALLOC_MAX_EXPERTS + 1];

constexpr int kMaxDevices = 64;
// Device address of g_routeScratch per device ordinal.  In host code the array's name is only a handle for the
// runtime, not an address a kernel could use, hence the lookup.  Fixed-size table: filling it allocates nothing.
uint32_t* g_scratchAddr[kMaxDevices] = {nullptr};

}  // namespace

extern "C" HcclResult HcclMoeExpertOffsetsNoAlloc(const int32_t* topkIdx, uint64_t nPairs, uint32_t nExperts, uint32_t* offsets,
                                                  hcclStream_t stream)
{
    using namespace hccl;
    CHK_PTR_NULL(topkIdx);
    CHK_PTR_NULL(offsets);
    if (nExperts == 0 || nExperts > HCCL_MOE_NOALLOC_MAX_EXPERTS) {
        HCCL_ERROR("HcclMoeExpertOffsetsNoAlloc: nExperts = %u is outside 1..%u, the size of the built-in scratch array; "
                   "use HcclMoeExpertOffsets for more experts", nExperts, HCCL_MOE_NOALLOC_MAX_EXPERTS);
        return HCCL_E_PARA;
    }
    int dev = -1;
    CHK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) { HCCL_ERROR("HcclMoeExpertOffsetsNoAlloc: device ordinal %d is not supported", dev); return HCCL_E_NOT_SUPPORT; }
    // Set-up, once per device and with that device current: resolve the device address of the array.  A concurrent
    // first call from another thread resolves the same value, so the unsynchronised store is harmless.
    uint32_t* scratch = g_scratchAddr[dev];
    if (scratch == nullptr) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_routeScratch);
        if (e != cudaSuccess || p == nullptr) {
            HCCL_ERROR("HcclMoeExpertOffsetsNoAlloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return HCCL_E_RUNTIME;
        }
        scratch = static_cast<uint32_t*>(p);
        g_scratchAddr[dev] = scratch;
    }
    // The tail of the array (beyond nExperts) holds the ticket of the widest layout; this call's ticket sits right
    // after its own counters, as the kernel expects, and is zero like the rest of the array between calls.
    MoeExpertOffsetsKernel<<<MoeExpertOffsetsBlocks(nPairs), 256, 0, (cudaStream_t)stream>>>(topkIdx, nPairs, nExperts, scratch, offsets);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("HcclMoeExpertOffsetsNoAlloc: launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}
