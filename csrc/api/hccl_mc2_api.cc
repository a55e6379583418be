// C entry points of the MC2 API: the op-args object and resource context of
// HCCL's hccl_mc2.h (behaviour: src/common/hccl_mc2.cc:39-167 - alloc / free /
// setters with range checks, engine restricted to the SM-driven engines, the
// context is created once per (communicator, op type) and cached), plus the
// fused operators themselves.
#include <cstring>
#include <mutex>
#include "../core/comm.h"
#include "../core/log.h"
#include "../kernels/dev_types.h"
#include "../kernels/mc2_launch.h"
#include "../ops/param_check.h"
#include "hccl/hccl_mc2.h"

using namespace hccl;

namespace {
constexpr uint32_t kOpArgsMagic = 0x4b464341u;  // "KFCA"
struct KfcOpArgs {
    uint32_t magic;
    uint8_t srcDataType, dstDataType, commEngine, pad;
    uint32_t reduceType;
    uint64_t count;
    char algConfig[128];
};
KfcOpArgs* Args(void* p)
{
    KfcOpArgs* a = static_cast<KfcOpArgs*>(p);
    return (a && a->magic == kOpArgsMagic) ? a : nullptr;
}
}  // namespace

extern "C" {

HcclResult HcclKfcAllocOpArgs(void** opArgs)
{
    CHK_PTR_NULL(opArgs);
    KfcOpArgs* a = new KfcOpArgs();
    memset(a, 0, sizeof(*a));
    a->magic = kOpArgsMagic;
    a->srcDataType = a->dstDataType = (uint8_t)HCCL_DATA_TYPE_BFP16;
    a->reduceType = HCCL_REDUCE_SUM;
    a->commEngine = (uint8_t)HCCL_ENGINE_P2P;
    *opArgs = a;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcFreeOpArgs(void* opArgs)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    a->magic = 0;
    delete a;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetSrcDataType(void* opArgs, uint8_t t)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    if (!IsValidDataType((HcclDataType)t)) return HCCL_E_PARA;
    a->srcDataType = t;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetDstDataType(void* opArgs, uint8_t t)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    if (!IsValidDataType((HcclDataType)t)) return HCCL_E_PARA;
    a->dstDataType = t;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetReduceType(void* opArgs, uint32_t r)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    if (r >= HCCL_REDUCE_RESERVED) return HCCL_E_PARA;
    a->reduceType = r;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetCount(void* opArgs, uint64_t count)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    CHK_RET(CheckCount("HcclKfcOpArgsSetCount", count));
    a->count = count;
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetAlgConfig(void* opArgs, char* algConfig)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    CHK_PTR_NULL(algConfig);
    if (strnlen(algConfig, sizeof(a->algConfig)) >= sizeof(a->algConfig)) return HCCL_E_PARA;
    snprintf(a->algConfig, sizeof(a->algConfig), "%s", algConfig);
    return HCCL_SUCCESS;
}
HcclResult HcclKfcOpArgsSetCommEngine(void* opArgs, uint8_t engine)
{
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    // fused kernels move their own data with SM loads / stores: only the SM-driven engines qualify
    // (the reference admits AICPU / AIV only, hccl_mc2.cc:129-133)
    if (engine != HCCL_ENGINE_P2P && engine != HCCL_ENGINE_NVLS && engine != HCCL_ENGINE_AUTO) return HCCL_E_NOT_SUPPORT;
    a->commEngine = engine;
    return HCCL_SUCCESS;
}

HcclResult HcclCreateOpResCtx(HcclComm comm, uint8_t opType, void* opArgs, void** opResCtx)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(opResCtx);
    KfcOpArgs* a = Args(opArgs);
    if (!a) return HCCL_E_PTR;
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (c->hostComm) return HCCL_E_NOT_SUPPORT;
    switch ((HcclCMDType)opType) {
        case HCCL_CMD_ALLGATHER: case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_ALLREDUCE: case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: break;
        default: HCCL_ERROR("HcclCreateOpResCtx: op type %u has no fused form", opType); return HCCL_E_NOT_SUPPORT;
    }
    const std::string tag = "mc2_ctx_" + std::to_string(opType);
    std::vector<uint8_t> blob;
    if (c->ctx.Get(tag, &blob) && blob.size() == sizeof(void*)) {   // one context per (communicator, op type)
        memcpy(opResCtx, blob.data(), sizeof(void*));
        return HCCL_SUCCESS;
    }
    HcclMc2ResCtx h;
    memset(&h, 0, sizeof(h));
    h.magic = HCCL_MC2_CTX_MAGIC;
    h.rank = (uint32_t)c->rank;
    h.rankSize = (uint32_t)c->nRanks;
    h.opType = opType;
    h.stageBytes = c->layout().dataBytes;
    for (int q = 0; q < c->nRanks; ++q) {
        h.stage[q] = c->StageBase(q);
        h.flags[q] = c->dev().slab[q];
    }
    h.stageMulticast = c->StageMcBase();
    h.status = c->dev().status;
    h.timeoutNs = c->cfg.execTimeoutNs;
    void* d = nullptr;
    CHK_CUDA(cudaMalloc(&d, sizeof(h)));
    CHK_CUDA(cudaMemcpy(d, &h, sizeof(h), cudaMemcpyHostToDevice));
    blob.resize(sizeof(void*));
    memcpy(blob.data(), &d, sizeof(void*));
    c->ctx.Put(tag, blob);
    *opResCtx = d;
    return HCCL_SUCCESS;
}

HcclResult HcclMc2Matmul(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transA, int transB, hcclStream_t stream)
{
    return Mc2Matmul(a, b, out, m, n, k, transA, transB, (cudaStream_t)stream);
}
HcclResult HcclMc2AllGatherMatmul(const void* aShard, const void* b, void* out, void* gathered, uint64_t mPerRank, uint64_t n, uint64_t k,
                                  int transB, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    CHK_RET(c->CheckReady());
    std::lock_guard<std::mutex> lk(c->opMu);
    return Mc2AllGatherMatmul(c, aShard, b, out, gathered, mPerRank, n, k, transB, (cudaStream_t)stream);
}
HcclResult HcclMc2MatmulReduceScatter(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transB, HcclComm comm,
                                      hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    CHK_RET(c->CheckReady());
    std::lock_guard<std::mutex> lk(c->opMu);
    return Mc2MatmulReduceScatter(c, a, b, out, m, n, k, transB, (cudaStream_t)stream);
}
HcclResult HcclMc2MatmulAllReduce(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transB, HcclComm comm,
                                  hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    CHK_RET(c->CheckReady());
    std::lock_guard<std::mutex> lk(c->opMu);
    return Mc2MatmulAllReduce(c, a, b, out, m, n, k, transB, (cudaStream_t)stream);
}

}  // extern "C"
