// Allocation-free variant of HcclMoeExpertOffsets.
//
// This entry point has no counterpart in the HCCL reference; it exists for callers of this library that are not
// allowed to allocate device memory at the moment they need the routing offsets: code running under a memory
// budget that has already handed every byte to a framework's caching allocator, plugins loaded into a serving
// process whose operator forbids cudaMalloc after start-up, and code on a latency path where the implicit device
// synchronisation of cudaMalloc / cudaFree is not acceptable.
//
// HcclMoeExpertOffsets keeps its counters in a buffer it allocates with cudaMalloc on first use.  The variant below
// keeps them in a fixed array that is part of the library image, so it never calls cudaMalloc, cudaFree or any
// other allocating routine.  The price: every GPU that loads the library holds
// (HCCL_MOE_NOALLOC_MAX_EXPERTS + 1) * 4 bytes (16 KiB + 4 B) of device memory until the process exits, and the
// number of experts is capped at HCCL_MOE_NOALLOC_MAX_EXPERTS (a larger value is rejected with HCCL_E_PARA and a log
// line that names the limit).
//
// Behaviour to know about:
//   * The first call on a device looks up the device address of that array (once per device, with that device
//     current).  Make that first call outside any CUDA stream capture; later calls only launch one kernel.
//   * All calls on one device share the array.  The kernel leaves it zeroed when it finishes, which the next call
//     relies on; two calls that overlap on the GPU (different streams without ordering between them) race on the
//     counters and produce wrong offsets.  Order them on one stream or with events.
//   * Inputs and outputs are the caller's, exactly as for HcclMoeExpertOffsets: topkIdx [nPairs] int32 and
//     offsets [nExperts + 1] uint32 in device memory; ids outside [0, nExperts) are ignored.
#ifndef HCCL_B200_MOE_NOALLOC_H_
#define HCCL_B200_MOE_NOALLOC_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

#define HCCL_MOE_NOALLOC_MAX_EXPERTS 4096u

HcclResult HcclMoeExpertOffsetsNoAlloc(const int32_t* topkIdx, uint64_t nPairs, uint32_t nExperts, uint32_t* offsets, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_MOE_NOALLOC_H_
