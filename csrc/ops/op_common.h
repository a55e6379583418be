// Operator parameter model and the single execution entry used by every
// operator (role of OpParam, alg_param.h:758-861, and HcclExecOp,
// op_common.cc:1259).  Counts are in elements; V arrays are copied from the
// caller's host arrays at entry so the call can return before the kernel runs.
#pragma once
#include <cstdint>
#include <string>
#include <vector>
#include <cuda_runtime.h>
#include "../core/comm.h"
#include "../select/selector.h"
#include "hccl/hccl_types.h"

namespace hccl {

struct OpParam {
    HcclCMDType op = HCCL_CMD_INVALID;
    std::string tag;
    const void* send = nullptr;
    void* recv = nullptr;
    uint64_t count = 0;
    HcclDataType dtype = HCCL_DATA_TYPE_RESERVED;
    HcclDataType recvType = HCCL_DATA_TYPE_RESERVED;
    HcclReduceOp redOp = HCCL_REDUCE_RESERVED;
    uint32_t root = 0;
    std::vector<uint64_t> sendCounts, sdispls, recvCounts, rdispls;   // per rank, in elements
    uint64_t globalMaxBytes = 0;     // largest single pair transfer over ALL ranks when it is known (AlltoAll, AlltoAllVC)
    std::vector<HcclSendRecvItem> items;
    cudaStream_t stream = nullptr;
    bool isMc2 = false;
    // reductions fused with a cast and a scale (HcclAllReduceEx / HcclReduceScatterEx): the output holds elements of
    // outType, every reduced value is multiplied by scale before it is stored
    bool castScale = false;
    HcclDataType outType = HCCL_DATA_TYPE_RESERVED;
    float scale = 1.0f;
    std::string algName;             // filled by ExecOp: the algorithm that ran
};

HcclResult ExecOp(CommImpl* comm, OpParam& p);

// The two halves of ExecOp for callers that collect the calls of several ranks first (ranks emulated on one GPU):
// what this rank's call looks like to the selector, and selection + execution on the flag word all ranks share.
OpDesc DescribeCall(CommImpl* comm, const OpParam& p);
HcclResult ExecDescribed(CommImpl* comm, OpParam& p, OpDesc d, const uint32_t* presetAgreedFlags);
// Queues a collective of an emulated rank; once every rank of the group has one queued, combines their flag words and
// runs them all.  Returns the result of the calls it ran (success while others are still missing).
HcclResult EmuSubmitCollective(CommImpl* comm, const OpParam& p);

}  // namespace hccl
