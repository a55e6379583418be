// Expert-parallel MoE dispatch / combine: AlltoAllV fused with token permutation,
// block-scaled fp8 quantisation (dispatch) and the gate-weighted sum (combine).
// The expert-parallel group is the communicator; expert e lives on rank
// e / (nExperts / rankSize).
#ifndef HCCL_B200_MOE_H_
#define HCCL_B200_MOE_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    uint32_t nTokens;     // tokens on this rank
    uint32_t hidden;      // multiple of 128, at most 8192
    uint32_t topk;        // at most 8
    uint32_t nExperts;    // global, multiple of rankSize, at most 512
    uint32_t capacity;    // rows of the receive buffers on every rank
} HcclMoeConfig;

// x: [nTokens, hidden] bf16; topkIdx: [nTokens, topk] int32 global expert ids (negative = dropped), device memory.
// recvX [capacity, hidden] fp8 e4m3, recvScale [capacity, hidden / 128] fp32 and recvSrc [capacity] uint64 must come
// from HcclMemAlloc (peers write them).  Outputs in local device memory: recvOffsets [nExperts / rankSize + 1]
// (row range of each local expert; rows of one expert are ordered by source rank) and slotMap [nTokens * topk]
// (where every pair went; input of HcclMoeCombine).  If more rows arrive than `capacity` the communicator reports
// an asynchronous error and the surplus rows are dropped.
HcclResult HcclMoeDispatch(HcclComm comm, const void* x, const int32_t* topkIdx, const HcclMoeConfig* cfg, void* recvX, void* recvScale,
                           void* recvSrc, uint32_t* recvOffsets, uint64_t* slotMap, hcclStream_t stream);
// y: [capacity, hidden] bf16 expert outputs in the row order of recvX, from HcclMemAlloc (peers read it);
// topkWeight: [nTokens, topk] fp32 gate weights; out: [nTokens, hidden] bf16 = sum_k weight[t, k] * y[slot(t, k)].
HcclResult HcclMoeCombine(HcclComm comm, const void* y, const float* topkWeight, const uint64_t* slotMap, const HcclMoeConfig* cfg, void* out,
                          hcclStream_t stream);

// Local routing helper (no communicator): offsets[e] .. offsets[e + 1] is the row range of expert e when this
// rank's nPairs (token, expert) pairs are grouped by expert; offsets has nExperts + 1 entries in device memory.
// Ids outside [0, nExperts) are ignored.  Keeps a small device scratch buffer per GPU (allocated on first use);
// calls on one GPU must be ordered (same stream) because they share it.
HcclResult HcclMoeExpertOffsets(const int32_t* topkIdx, uint64_t nPairs, uint32_t nExperts, uint32_t* offsets, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_MOE_H_
