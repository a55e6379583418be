// Host interface of the MC2 (matmul + collective) kernels.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "../core/symmem.h"
#include "hccl/hccl_types.h"

namespace hccl {

class CommImpl;

// Per-communicator resources of the fused kernels: the device control block, tile flags (symmetric) and the
// exchange buffer for partial tiles (symmetric, two parities), grown on demand.
struct Mc2State {
    uint32_t* ctl = nullptr;            // device, zero-initialised
    SymSegment flags;                   // [nRanks][kMaxTiles] uint64
    SymSegment xchg;                    // 2 * parityBytes
    uint64_t xchgParityBytes = 0;
    void* resCtxDev = nullptr;          // device copy of HcclMc2ResCtx (HcclCreateOpResCtx)
    ~Mc2State();
};
constexpr int kMc2MaxTiles = 16384;
constexpr int kMc2AgBlocks = 8 * 512;   // arrival counters of the push-form AllGather: ranks x 128-row blocks per rank
constexpr int kMc2CtlWords = 16 + 8 * 512;

HcclResult Mc2Matmul(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transA, int transB,
                     cudaStream_t stream);
HcclResult Mc2AllGatherMatmul(CommImpl* comm, const void* aShard, const void* b, void* out, void* gathered, uint64_t mPerRank,
                              uint64_t n, uint64_t k, int transB, cudaStream_t stream);
HcclResult Mc2MatmulReduceScatter(CommImpl* comm, const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k,
                                  int transB, cudaStream_t stream);
HcclResult Mc2MatmulAllReduce(CommImpl* comm, const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k,
                              int transB, cudaStream_t stream);
// Collective: makes sure the exchange buffer can hold `parityBytes` per parity (reallocates symmetric memory).
HcclResult Mc2EnsureState(CommImpl* comm, uint64_t parityBytes);

}  // namespace hccl
