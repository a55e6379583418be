// Host interface of the MoE dispatch / combine kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cuda_bf16.h>
#include "dev_types.h"
#include "launch.h"

namespace hccl {

constexpr int kMoeMaxExperts = 512;
constexpr int kMoeMaxTopk = 8;
constexpr size_t kMoeTableBytes = (size_t)kMaxBlocks * kMaxDevRanks * kMoeMaxExperts * sizeof(uint32_t);

struct MoeDispatchArgs {
    const __nv_bfloat16* x;            // [nTokens, hidden]
    const int32_t* topkIdx;            // [nTokens, topk] global expert ids (negative = dropped)
    const uint32_t* counts;            // [nExperts] pairs per expert on this rank
    const uint32_t* pos;               // [nTokens * topk] position of the pair among this rank's pairs of that expert
    uint64_t* slotMap;                 // [nTokens * topk] out: (destination rank << 32) | slot
    uint32_t* recvOffsets;             // [nExperts / nRanks + 1] out: where each local expert starts in the receive buffer
    uint32_t* table[kMaxDevRanks];     // count exchange table of every rank (symmetric)
    uint8_t* recvX[kMaxDevRanks];      // [capacity, hidden] fp8 e4m3 (symmetric)
    float* recvScale[kMaxDevRanks];    // [capacity, hidden / 128] (symmetric)
    uint64_t* recvSrc[kMaxDevRanks];   // [capacity] (source rank << 32) | (token * topk + k) (symmetric)
    int nTokens, hidden, topk, nExperts;
    uint32_t capacity;
};

struct MoeCombineArgs {
    const __nv_bfloat16* y[kMaxDevRanks];   // expert outputs [capacity, hidden] of every rank (symmetric)
    const float* topkWeight;                // [nTokens, topk]
    const uint64_t* slotMap;                // from dispatch
    __nv_bfloat16* out;                     // [nTokens, hidden]
    int nTokens, hidden, topk;
    uint32_t capacity;
};

HcclResult LaunchMoeCount(const int32_t* topkIdx, int nPairs, int nExperts, uint32_t* counts, uint32_t* pos, cudaStream_t stream);
HcclResult LaunchMoeDispatch(const LaunchTarget& t, const MoeDispatchArgs& a, int nBlocks);
HcclResult LaunchMoeCombine(const LaunchTarget& t, const MoeCombineArgs& a, int nBlocks);

}  // namespace hccl
