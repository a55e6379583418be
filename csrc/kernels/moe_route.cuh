// Expert histogram + exclusive scan for MoE routing: from the [tokens, topk]
// expert ids of this rank, the row range every expert's tokens occupy when the
// (token, expert) pairs are grouped by expert (what a grouped GEMM consumes).
// The kernel needs `nExperts + 1` 32-bit words of scratch that are zero when it
// starts: per-expert counters and an exit ticket.  Blocks add their pairs to
// the counters; the last block to finish turns the counters into offsets and
// leaves the scratch zeroed again for the next call.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace hccl {

static __global__ void MoeExpertOffsetsKernel(const int32_t* __restrict__ topkIdx, uint64_t nPairs, uint32_t nExperts,
                                              uint32_t* __restrict__ scratch, uint32_t* __restrict__ offsets)
{
    uint32_t* counters = scratch;
    uint32_t* ticket = scratch + nExperts;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nPairs; i += (uint64_t)gridDim.x * blockDim.x) {
        const int32_t e = topkIdx[i];
        if (e >= 0 && (uint32_t)e < nExperts) atomicAdd(&counters[e], 1u);
    }
    __shared__ bool s_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(ticket, 1u) == gridDim.x - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x == 0) {
        uint32_t run = 0;
        for (uint32_t e = 0; e < nExperts; ++e) {
            const uint32_t c = *reinterpret_cast<volatile uint32_t*>(&counters[e]);
            offsets[e] = run;
            run += c;
            counters[e] = 0;          // the scratch is zero again when the kernel ends
        }
        offsets[nExperts] = run;
        *ticket = 0;
    }
}

inline int MoeExpertOffsetsBlocks(uint64_t nPairs)
{
    uint64_t b = (nPairs + 1023) / 1024;
    return (int)(b < 1 ? 1 : (b > 64 ? 64 : b));
}

}  // namespace hccl
