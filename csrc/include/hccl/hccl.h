// Collective and point-to-point operator entry points of hccl_b200.
//
// Names, argument order and semantics follow include/hccl.h:36-266 of HCCL
// (aclrtStream becomes a CUDA stream).  Every call is asynchronous with respect
// to the host and ordered on `stream`; counts are in elements.
#ifndef HCCL_B200_H_
#define HCCL_B200_H_

#include "hccl_types.h"
#include "hccl_comm.h"

#ifdef __cplusplus
extern "C" {
#endif

HcclResult HcclAllReduce(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                         HcclComm comm, hcclStream_t stream);
HcclResult HcclBroadcast(void* buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm,
                         hcclStream_t stream);
HcclResult HcclReduceScatter(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType,
                             HcclReduceOp op, HcclComm comm, hcclStream_t stream);
// sendCounts / sendDispls: host arrays of uint64_t, one entry per rank.
HcclResult HcclReduceScatterV(void* sendBuf, const void* sendCounts, const void* sendDispls, void* recvBuf,
                              uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                              hcclStream_t stream);
HcclResult HcclScatter(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root,
                       HcclComm comm, hcclStream_t stream);
HcclResult HcclAllGather(void* sendBuf, void* recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm,
                         hcclStream_t stream);
HcclResult HcclAllGatherV(void* sendBuf, uint64_t sendCount, void* recvBuf, const void* recvCounts,
                          const void* recvDispls, HcclDataType dataType, HcclComm comm, hcclStream_t stream);
HcclResult HcclSend(void* sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm,
                    hcclStream_t stream);
HcclResult HcclRecv(void* recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm,
                    hcclStream_t stream);
// sendCountMatrix: host uint64_t[rankSize*rankSize], row i = what rank i sends to each rank.
HcclResult HcclAlltoAllVC(const void* sendBuf, const void* sendCountMatrix, HcclDataType sendType,
                          const void* recvBuf, HcclDataType recvType, HcclComm comm, hcclStream_t stream);
HcclResult HcclAlltoAllV(const void* sendBuf, const void* sendCounts, const void* sdispls, HcclDataType sendType,
                         const void* recvBuf, const void* recvCounts, const void* rdispls, HcclDataType recvType,
                         HcclComm comm, hcclStream_t stream);
HcclResult HcclAlltoAll(const void* sendBuf, uint64_t sendCount, HcclDataType sendType, const void* recvBuf,
                        uint64_t recvCount, HcclDataType recvType, HcclComm comm, hcclStream_t stream);
HcclResult HcclReduce(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op,
                      uint32_t root, HcclComm comm, hcclStream_t stream);
HcclResult HcclBatchSendRecv(HcclSendRecvItem* sendRecvInfo, uint32_t itemNum, HcclComm comm, hcclStream_t stream);
HcclResult HcclBarrier(HcclComm comm, hcclStream_t stream);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_H_
