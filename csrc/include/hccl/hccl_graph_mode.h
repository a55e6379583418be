// Graph-mode twins of the operators.
//
// A graph builder does not hold communicator handles: it knows a communication
// group by NAME, gives every operator node a TAG, and sizes the node's resources
// (scratch, extra streams) before the graph runs.  The reference exposes that
// as HcclAllReduceGraphMode etc. (all_reduce.cc:58) with a ResPackGraphMode
// (alg_param.h:928-933) and the HcclCalcOpRes*GraphMode family
// (interface_graph_mode/calc_resource_graph_mode.cc:51-633).
//
// Here every operator is one stream-ordered kernel on the caller's stream that
// works in the communicator's own staging slab, so a node needs no scratch of
// its own and no extra streams; a resource pack is accepted and checked, and the
// query reports what a node will use.  The calls can be captured in a CUDA graph.
//
// A group name resolves to the communicator of that name in this process.  When
// several ranks of the group live in one process (threads as ranks), each thread
// first binds its communicator with HcclGroupBindThread.
#ifndef HCCL_B200_GRAPH_MODE_H
#define HCCL_B200_GRAPH_MODE_H
#include "hccl.h"
#include <stdbool.h>
#include "hccl_ext.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct {
    uint32_t size;                 // sizeof(HcclResPackGraphMode), for versioning
    void* scratch;                 // optional: unused by this library's operators
    uint64_t scratchBytes;
    hcclStream_t* slaveStreams;    // optional: unused, operators stay on the caller's stream
    uint32_t slaveStreamNum;
} HcclResPackGraphMode;

// Group lookup.  HcclGroupGetComm fails with HCCL_E_NOT_FOUND for an unknown name and with HCCL_E_PARA when the name
// is ambiguous in this process and the calling thread has bound none of the candidates.
HcclResult HcclGroupGetComm(const char* group, HcclComm* comm);
HcclResult HcclGroupBindThread(HcclComm comm);
HcclResult HcclGroupUnbindThread(const char* group);

// What a node of this operator will use (the role of HcclCalcOpResOffline / ...GraphMode).
HcclResult HcclCalcOpResGraphMode(const char* group, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp,
                                  HcclOpResource* res);

// The same for a group that exists (online; `registered` != 0: the node's buffers come from HcclMemAlloc), and for a
// box that is only described (offline: no communicator, no device; nRanks GPUs behind one NVSwitch, nvls != 0 when the
// switch reduces, bufferBytes = the staging slab, 0 for the configured default).  Reference: HcclCalcOpResOnline /
// OfflineGraphMode (interface_graph_mode/calc_resource_graph_mode.cc).
HcclResult HcclCalcOpResOnlineGraphMode(const char* group, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp, int registered,
                                        HcclOpResource* res);
HcclResult HcclCalcOpResOfflineGraphMode(uint32_t nRanks, int nvls, uint64_t bufferBytes, HcclCMDType op, uint64_t count, HcclDataType dataType,
                                         HcclReduceOp reduceOp, int registered, HcclOpResource* res);

// A node described field by field, for graph builders that assemble an operator before any group exists (reference:
// HcclCreateOpParamGraphMode / HcclSetOpParamGraphMode<Field> / HcclCalcOpResOnlineGraphMode(opParam, ...) /
// HcclSetAivSelectOpParamGraphMode, calc_resource_graph_mode.h).  Defaults: 8 ranks, switch reduction available, the
// configured slab, fp32, sum, ordinary buffers, no block limit.  The operator is named as the graph names it:
// "AllReduce", "HcomAllReduce", "allreduce", ... (prefix and case are ignored).  The vector cores of the reference
// correspond to thread blocks here: a block limit caps the grid of the node's kernels.
typedef struct HcclOpParamGraphMode HcclOpParamGraphMode;
HcclResult HcclCreateOpParamGraphMode(HcclOpParamGraphMode** opParam);
HcclResult HcclDestroyOpParamGraphMode(HcclOpParamGraphMode* opParam);
HcclResult HcclSetOpParamGraphModeOpType(HcclOpParamGraphMode* opParam, const char* opType);
HcclResult HcclSetOpParamGraphModeDataCount(HcclOpParamGraphMode* opParam, uint64_t dataCount);
HcclResult HcclSetOpParamGraphModeRankSize(HcclOpParamGraphMode* opParam, uint32_t rankSize);
HcclResult HcclSetOpParamGraphModeHCCLBufferSize(HcclOpParamGraphMode* opParam, uint64_t bufferBytes);
HcclResult HcclSetOpParamGraphModeDataType(HcclOpParamGraphMode* opParam, HcclDataType dataType);
HcclResult HcclSetOpParamGraphModeReduceType(HcclOpParamGraphMode* opParam, HcclReduceOp reduceOp);
HcclResult HcclSetOpParamGraphModeRegistered(HcclOpParamGraphMode* opParam, int registered, int switchReduces);
HcclResult HcclSetOpParamGraphModeBlockLimit(HcclOpParamGraphMode* opParam, uint32_t blockLimit);
// opMemSize: staging bytes of the slab one launch uses; streamNum: 1; taskNum: kernel launches; blockNum: grid size.
HcclResult HcclCalcOpResOpParamGraphMode(const HcclOpParamGraphMode* opParam, uint64_t* opMemSize, uint32_t* streamNum, uint32_t* taskNum,
                                         uint32_t* blockNum, char algName[128]);
// Which algorithm a node of an existing group will run and whether it runs on the device engines (the reference's
// HcclSelectAlgGraphMode with its AIV flag); blockLimit 0 = the group's own.
HcclResult HcclSelectAlgGraphMode(const char* group, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType, uint32_t blockLimit,
                                  bool* onDevice, char algName[128]);
// The grid a node of an existing group will launch (the reference's HcclCalcAivCoreNumGraphMode).
HcclResult HcclCalcBlockNumGraphMode(const char* group, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType, uint32_t blockLimit,
                                     uint32_t* numBlocks);
// What a fused kernel of the graph needs to talk to the group without going through an operator call: *commContext
// receives a DEVICE pointer to the group's HcclMc2ResCtx for opType (peer tables, flag rows, multicast alias;
// hccl_mc2.h), *len its size.  The reference hands a graph's fused node its communicator context the same way
// (HcclGetAlgExecParamGraphMode); the tag names the node in the logs.  Device communicators only.
HcclResult HcclGetAlgExecParamGraphMode(const char* tag, const char* group, uint64_t count, HcclCMDType opType, HcclDataType dataType, HcclReduceOp op,
                                        void** commContext, uint64_t* len);
// Caps the grids of every later operator of the group (1..128; 0 lifts the cap).  Reference: HcclSetAivCoreLimitGraphMode.
HcclResult HcclSetBlockLimitGraphMode(const char* group, uint32_t blockLimit);

HcclResult HcclAllReduceGraphMode(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, const char* group,
                                  const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclBroadcastGraphMode(void* buf, uint64_t count, HcclDataType dataType, uint32_t root, const char* group, const char* tag,
                                  const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclReduceScatterGraphMode(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op,
                                      const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclAllGatherGraphMode(void* sendBuf, void* recvBuf, uint64_t sendCount, HcclDataType dataType, const char* group,
                                  const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclReduceGraphMode(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root,
                               const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclScatterGraphMode(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, const char* group,
                                const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclAlltoAllGraphMode(const void* sendBuf, uint64_t sendCount, HcclDataType sendType, const void* recvBuf, uint64_t recvCount,
                                 HcclDataType recvType, const char* group, const char* tag, const HcclResPackGraphMode* res,
                                 hcclStream_t stream);
// Counts and displacements: host arrays of uint64_t, as in the operators themselves.
HcclResult HcclAllGatherVGraphMode(void* sendBuf, void* recvBuf, uint64_t sendCount, const void* recvCounts, const void* recvDispls,
                                   HcclDataType dataType, const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclReduceScatterVGraphMode(void* sendBuf, const void* sendCounts, const void* sendDispls, void* recvBuf, uint64_t recvCount,
                                       HcclDataType dataType, HcclReduceOp op, const char* group, const char* tag, const HcclResPackGraphMode* res,
                                       hcclStream_t stream);
HcclResult HcclAlltoAllVGraphMode(const void* sendBuf, const void* sendCounts, const void* sdispls, HcclDataType sendType, const void* recvBuf,
                                  const void* recvCounts, const void* rdispls, HcclDataType recvType, const char* group, const char* tag,
                                  const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclAlltoAllVCGraphMode(const void* sendBuf, const void* sendCountMatrix, HcclDataType sendType, const void* recvBuf,
                                   HcclDataType recvType, const char* group, const char* tag, const HcclResPackGraphMode* res,
                                   hcclStream_t stream);
HcclResult HcclSendGraphMode(void* sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, const char* group, const char* tag,
                             const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclRecvGraphMode(void* recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, const char* group, const char* tag,
                             const HcclResPackGraphMode* res, hcclStream_t stream);
HcclResult HcclBarrierGraphMode(const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif
