// Communicator management API of hccl_b200.
//
// HCCL keeps these entry points in its HCOMM half (they are only *used* by the
// operator repository: examples/02_collectives/01_allreduce/main.cc:76-123,
// test/st/algorithm/testcase/all_reduce_testcase.cc:89); this library supplies
// both halves.  One process (or thread) drives one GPU.
#ifndef HCCL_B200_COMM_H_
#define HCCL_B200_COMM_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

// Rank 0 creates the rendezvous endpoint; the bytes are sent out of band to
// every rank, which passes them to HcclCommInitRootInfo.
HcclResult HcclGetRootInfo(HcclRootInfo* rootInfo);
HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo* rootInfo, uint32_t rank, HcclComm* comm);
HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo* rootInfo, uint32_t rank,
                                      const HcclCommConfig* config, HcclComm* comm);
// JSON rank table ("server_list"/"device" entries with rank_id, device_id and a
// "root" {ip, port}); see docs/ranktable.md.
HcclResult HcclCommInitClusterInfo(const char* clusterInfo, uint32_t rank, HcclComm* comm);
HcclResult HcclCommInitClusterInfoConfig(const char* clusterInfo, uint32_t rank, const HcclCommConfig* config,
                                         HcclComm* comm);
// Single process, one communicator per listed device.  With HCCL_B200_EMULATE=1
// (or when every listed device is the same GPU) the ranks share one GPU and every
// collective runs as ONE cooperative kernel over all ranks' data.
HcclResult HcclCommInitAll(uint32_t ndev, const int32_t* devices, HcclComm* comms);
HcclResult HcclCommDestroy(HcclComm comm);

HcclResult HcclGetRankSize(HcclComm comm, uint32_t* rankSize);
HcclResult HcclGetRankId(HcclComm comm, uint32_t* rank);
HcclResult HcclGetCommName(HcclComm comm, char* commName);  // buffer of >= 128 bytes
HcclResult HcclCommGetStatus(HcclComm comm, HcclCommStatus* status);
HcclResult HcclCommSuspend(HcclComm comm);
HcclResult HcclCommResume(HcclComm comm);
// Last asynchronous device-side error (bounded wait that ran out, ...).
HcclResult HcclCommGetAsyncError(HcclComm comm, HcclResult* asyncError);
const char* HcclGetErrorString(HcclResult code);

// Staging slab of the communicator (device pointer + size in bytes).
HcclResult HcclGetHcclBuffer(HcclComm comm, void** buffer, uint64_t* size);

// Symmetric (zero-copy) memory: collective calls, every rank passes the same size.
HcclResult HcclMemAlloc(HcclComm comm, uint64_t size, void** devPtr);
HcclResult HcclMemFree(HcclComm comm, void* devPtr);
// Registration of a buffer the caller allocated itself (cudaMalloc, or a framework allocator on top of it): collective,
// every rank passes its own buffer of the same size and later uses the same offsets inside it.  Operators then read
// and write it in place on the peers (peer-to-peer kernels, no staging copies; no switch reduction: for that use
// HcclMemAlloc).  The reference's counterpart is the registration of user buffers for zero copy
// (RegGraphModeBuffers, op_common.cc:2724).  Deregister before freeing the buffer.
HcclResult HcclCommRegister(HcclComm comm, void* devPtr, uint64_t size);
HcclResult HcclCommDeregister(HcclComm comm, void* devPtr);
// Peer address of `localPtr` (inside a symmetric allocation) on `peerRank`,
// mapped into this process; and the multicast alias (NULL when NVLS is off).
HcclResult HcclCommSymWinGet(HcclComm comm, const void* localPtr, uint32_t peerRank, void** peerPtr);
HcclResult HcclCommSymWinGetMulticast(HcclComm comm, const void* localPtr, void** mcPtr);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_COMM_H_
