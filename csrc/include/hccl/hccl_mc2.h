// MC2 (matmul + collective fusion) resource API and the fused operators.
//
// HCCL only publishes the resource-context half (include/hccl_mc2.h:26-94: an
// op-args object plus HcclCreateOpResCtx, implemented in
// src/common/hccl_mc2.cc:39-167); its fused kernels live in another package.
// Here the same resource API returns a device-readable context (peer tables,
// flag rows, multicast alias) and the fused AllGather->Matmul,
// Matmul->ReduceScatter and Matmul->AllReduce kernels are part of the library.
#ifndef HCCL_B200_MC2_H_
#define HCCL_B200_MC2_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclKfcAllocOpArgs(void** opArgs);
HcclResult HcclKfcFreeOpArgs(void* opArgs);
HcclResult HcclKfcOpArgsSetSrcDataType(void* opArgs, uint8_t srcDataType);
HcclResult HcclKfcOpArgsSetDstDataType(void* opArgs, uint8_t dstDataType);
HcclResult HcclKfcOpArgsSetReduceType(void* opArgs, uint32_t reduceType);
HcclResult HcclKfcOpArgsSetCount(void* opArgs, uint64_t count);
HcclResult HcclKfcOpArgsSetAlgConfig(void* opArgs, char* algConfig);
HcclResult HcclKfcOpArgsSetCommEngine(void* opArgs, uint8_t commEngine);
// *opResCtx receives a DEVICE pointer to an HcclMc2ResCtx that stays valid until
// the communicator is destroyed.
HcclResult HcclCreateOpResCtx(HcclComm comm, uint8_t opType, void* opArgs, void** opResCtx);

// Layout of the context a fused kernel reads.
typedef struct {
    uint32_t magic;
    uint32_t rank;
    uint32_t rankSize;
    uint32_t opType;
    uint64_t stageBytes;
    void* stage[HCCL_MAX_DEVICE_RANKS];      // peers' staging slabs mapped here
    void* flags[HCCL_MAX_DEVICE_RANKS];      // peers' flag areas mapped here
    void* stageMulticast;                    // NULL when NVLS is off
    void* status;                            // host-mapped status block
    uint64_t timeoutNs;
} HcclMc2ResCtx;
#define HCCL_MC2_CTX_MAGIC 0x4d433242u

// ---- fused operators (bf16 in, fp32 accumulate, bf16 out) -------------------
// Shapes are row-major.  `transB` = 0: B is [K, N]; 1: B is [N, K] (a Linear
// weight).  All device buffers that peers touch must come from HcclMemAlloc.
//
// AllGather->Matmul: every rank holds aShard [mPerRank, K]; computes
//   out[rankSize*mPerRank, N] = AllGather(aShard) x B.  `gathered` (optional,
//   symmetric, [rankSize*mPerRank, K]) also receives the gathered activations.
HcclResult HcclMc2AllGatherMatmul(const void* aShard, const void* b, void* out, void* gathered, uint64_t mPerRank,
                                  uint64_t n, uint64_t k, int transB, HcclComm comm, hcclStream_t stream);
// Matmul->ReduceScatter: out[m/rankSize, N] = ReduceScatter_rows(A[m,K] x B).
HcclResult HcclMc2MatmulReduceScatter(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k,
                                      int transB, HcclComm comm, hcclStream_t stream);
// Matmul->AllReduce: out[m, N] = AllReduce(A[m,K] x B).
HcclResult HcclMc2MatmulAllReduce(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k,
                                  int transB, HcclComm comm, hcclStream_t stream);
// Plain local GEMM on the same tcgen05 pipeline (C = op(A) x op(B)); transA = 1: A is [K, M].
HcclResult HcclMc2Matmul(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transA,
                         int transB, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_MC2_H_
