// Operator entry points: parameter checks, tag, OpParam fill, then ExecOp.
//
// Per-operator behaviour follows the reference entry files: count == 0 returns
// success without touching the device (all_reduce.cc:41); pointer, count, data
// type and reduce-op checks happen before anything else (all_reduce.cc:111-137);
// the V operators read their host uint64 arrays at entry (all_to_all_v.cc:121-128)
// and AlltoAll / AlltoAllVC are lowered to the AlltoAllV form
// (all_to_all_v.cc:62-73, :424-448); BatchSendRecv copies its item list
// (batch_send_recv.cc:99-110).
#include <algorithm>
#include <cstring>
#include <map>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <mutex>
#include <new>
#include <string>
#include "../core/log.h"
#include "../core/plan_cache.h"
#include "../kernels/dev_types.h"
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "hccl/hccl.h"
#include "hccl/hccl_graph_mode.h"
#include "hccl/hccl_mc2.h"

using namespace hccl;

namespace {

CommImpl* C(HcclComm comm) { return static_cast<CommImpl*>(comm); }

// Tag of the graph node that is being issued on this thread (graph-mode twins), else null.
thread_local const char* g_graphTag = nullptr;

HcclResult Finish(CommImpl* c, OpParam& p)
{
    HcclResult r = ExecOp(c, p);
    if (!p.algName.empty()) c->ctx.Put("last_alg", std::vector<uint8_t>(p.algName.begin(), p.algName.end()));
    return r;
}

void Fill(OpParam& p, HcclCMDType op, CommImpl* c, const void* send, void* recv, uint64_t count, HcclDataType dt, HcclReduceOp rop,
          uint32_t root, hcclStream_t stream)
{
    p.op = op;
    p.tag = g_graphTag ? std::string(g_graphTag) : std::string(CmdName(op)) + "_" + c->name;
    p.send = send;
    p.recv = recv;
    p.count = count;
    p.dtype = dt;
    p.recvType = dt;
    p.redOp = rop;
    p.root = root;
    p.stream = (cudaStream_t)stream;
}

void ReadU64(const void* hostArray, uint32_t n, std::vector<uint64_t>* out)
{
    const uint64_t* a = static_cast<const uint64_t*>(hostArray);
    out->assign(a, a + n);
}

}  // namespace

extern "C" {

HcclResult HcclAllReduce(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                         hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckCount("HcclAllReduce", count));
    CHK_RET(CheckDataType("HcclAllReduce", dataType, true, false));
    CHK_RET(CheckReduceOp("HcclAllReduce", dataType, op));
    OpParam p;
    Fill(p, HCCL_CMD_ALLREDUCE, C(comm), sendBuf, recvBuf, count, dataType, op, 0, stream);
    return Finish(C(comm), p);
}

HcclResult HcclBroadcast(void* buf, uint64_t count, HcclDataType dataType, uint32_t root, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(buf);
    CHK_RET(CheckCount("HcclBroadcast", count));
    CHK_RET(CheckDataType("HcclBroadcast", dataType, false, false));
    CHK_RET(CheckRank("HcclBroadcast", "root", root, (uint32_t)C(comm)->nRanks));
    OpParam p;
    Fill(p, HCCL_CMD_BROADCAST, C(comm), buf, buf, count, dataType, HCCL_REDUCE_RESERVED, root, stream);
    return Finish(C(comm), p);
}

HcclResult HcclReduceScatter(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, HcclComm comm,
                             hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (recvCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckCount("HcclReduceScatter", recvCount * (uint64_t)C(comm)->nRanks));
    CHK_RET(CheckDataType("HcclReduceScatter", dataType, true, true));
    CHK_RET(CheckReduceOp("HcclReduceScatter", dataType, op));
    OpParam p;
    Fill(p, HCCL_CMD_REDUCE_SCATTER, C(comm), sendBuf, recvBuf, recvCount, dataType, op, 0, stream);
    return Finish(C(comm), p);
}

// ---- reductions fused with a cast and a scale ------------------------------------------------------------------
namespace {
bool IsCastType(HcclDataType t) { return t == HCCL_DATA_TYPE_FP32 || t == HCCL_DATA_TYPE_BFP16 || t == HCCL_DATA_TYPE_FP16; }
float LoadAs(const void* p, HcclDataType t, uint64_t i)
{
    switch (t) {
        case HCCL_DATA_TYPE_FP32: return static_cast<const float*>(p)[i];
        case HCCL_DATA_TYPE_BFP16: return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
        default: return __half2float(static_cast<const __half*>(p)[i]);
    }
}
void StoreAs(void* p, HcclDataType t, uint64_t i, float v)
{
    switch (t) {
        case HCCL_DATA_TYPE_FP32: static_cast<float*>(p)[i] = v; break;
        case HCCL_DATA_TYPE_BFP16: static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v); break;
        default: static_cast<__half*>(p)[i] = __float2half_rn(v); break;
    }
}
HcclResult CheckEx(const char* what, HcclDataType inType, HcclDataType outType, float scale)
{
    if (!IsCastType(inType) || !IsCastType(outType)) {
        HCCL_ERROR("%s: input and output types must be fp32, bf16 or fp16 (got %s -> %s)", what, DataTypeName(inType), DataTypeName(outType));
        return HCCL_E_NOT_SUPPORT;
    }
    if (!(scale == scale) || scale == 0.0f) { HCCL_ERROR("%s: scale must be a non-zero number", what); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}
}  // namespace

HcclResult HcclAllReduceEx(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType inType, HcclDataType outType, HcclReduceOp op, float scale,
                           HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (count == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckCount("HcclAllReduceEx", count));
    CHK_RET(CheckEx("HcclAllReduceEx", inType, outType, scale));
    CHK_RET(CheckReduceOp("HcclAllReduceEx", inType, op));
    if (inType == outType && scale == 1.0f) return HcclAllReduce(sendBuf, recvBuf, count, inType, op, comm, stream);
    CommImpl* c = C(comm);
    if (c->hostComm || c->nRanks == 1) {
        // host engine (and the single-rank shortcut): the plain operator, then cast and scale on the host / by a copy kernel
        if (c->hostComm) {
            std::vector<char> tmp(count * DataTypeSize(inType));
            CHK_RET(HcclAllReduce(sendBuf, tmp.data(), count, inType, op, comm, stream));
            for (uint64_t i = 0; i < count; ++i) StoreAs(recvBuf, outType, i, LoadAs(tmp.data(), inType, i) * scale);
            return HCCL_SUCCESS;
        }
        HCCL_ERROR("HcclAllReduceEx needs more than one rank on a device communicator");
        return HCCL_E_NOT_SUPPORT;
    }
    OpParam p;
    Fill(p, HCCL_CMD_ALLREDUCE, c, sendBuf, recvBuf, count, inType, op, 0, stream);
    p.castScale = true;
    p.outType = outType;
    p.scale = scale;
    return Finish(c, p);
}

HcclResult HcclReduceScatterEx(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType inType, HcclDataType outType, HcclReduceOp op,
                               float scale, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (recvCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CommImpl* c = C(comm);
    CHK_RET(CheckCount("HcclReduceScatterEx", recvCount * (uint64_t)c->nRanks));
    CHK_RET(CheckEx("HcclReduceScatterEx", inType, outType, scale));
    CHK_RET(CheckReduceOp("HcclReduceScatterEx", inType, op));
    if (inType == outType && scale == 1.0f) return HcclReduceScatter(sendBuf, recvBuf, recvCount, inType, op, comm, stream);
    if (c->hostComm) {
        std::vector<char> tmp(recvCount * DataTypeSize(inType));
        CHK_RET(HcclReduceScatter(sendBuf, tmp.data(), recvCount, inType, op, comm, stream));
        for (uint64_t i = 0; i < recvCount; ++i) StoreAs(recvBuf, outType, i, LoadAs(tmp.data(), inType, i) * scale);
        return HCCL_SUCCESS;
    }
    if (c->nRanks == 1) { HCCL_ERROR("HcclReduceScatterEx needs more than one rank on a device communicator"); return HCCL_E_NOT_SUPPORT; }
    OpParam p;
    Fill(p, HCCL_CMD_REDUCE_SCATTER, c, sendBuf, recvBuf, recvCount, inType, op, 0, stream);
    p.castScale = true;
    p.outType = outType;
    p.scale = scale;
    return Finish(c, p);
}

HcclResult HcclReduceScatterV(void* sendBuf, const void* sendCounts, const void* sendDispls, void* recvBuf, uint64_t recvCount,
                              HcclDataType dataType, HcclReduceOp op, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(sendCounts);
    CHK_PTR_NULL(sendDispls);
    CommImpl* c = C(comm);
    CHK_RET(CheckDataType("HcclReduceScatterV", dataType, true, false));
    CHK_RET(CheckReduceOp("HcclReduceScatterV", dataType, op));
    OpParam p;
    Fill(p, HCCL_CMD_REDUCE_SCATTER_V, c, sendBuf, recvBuf, recvCount, dataType, op, 0, stream);
    ReadU64(sendCounts, (uint32_t)c->nRanks, &p.sendCounts);
    ReadU64(sendDispls, (uint32_t)c->nRanks, &p.sdispls);
    uint64_t total = 0;
    for (int q = 0; q < c->nRanks; ++q) {
        CHK_RET(CheckCount("HcclReduceScatterV", p.sendCounts[(size_t)q]));
        CHK_RET(CheckCount("HcclReduceScatterV", p.sdispls[(size_t)q] + p.sendCounts[(size_t)q]));
        total += p.sendCounts[(size_t)q];
    }
    if (p.sendCounts[(size_t)c->rank] != recvCount) {
        ReportInputError("EI0003", "HcclReduceScatterV", "recvCount", std::to_string(recvCount), "sendCounts[rank]");
        return HCCL_E_PARA;
    }
    if (total == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    if (recvCount) CHK_PTR_NULL(recvBuf);
    return Finish(c, p);
}

HcclResult HcclScatter(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, HcclComm comm,
                       hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (recvCount == 0) return HCCL_SUCCESS;
    CommImpl* c = C(comm);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckRank("HcclScatter", "root", root, (uint32_t)c->nRanks));
    if ((uint32_t)c->rank == root) CHK_PTR_NULL(sendBuf);
    CHK_RET(CheckCount("HcclScatter", recvCount * (uint64_t)c->nRanks));
    CHK_RET(CheckDataType("HcclScatter", dataType, false, false));
    OpParam p;
    // only the root's send buffer is read; the other ranks pass anything
    Fill(p, HCCL_CMD_SCATTER, c, (uint32_t)c->rank == root ? sendBuf : nullptr, recvBuf, recvCount, dataType, HCCL_REDUCE_RESERVED, root, stream);
    return Finish(c, p);
}

HcclResult HcclAllGather(void* sendBuf, void* recvBuf, uint64_t sendCount, HcclDataType dataType, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (sendCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckCount("HcclAllGather", sendCount * (uint64_t)C(comm)->nRanks));
    CHK_RET(CheckDataType("HcclAllGather", dataType, false, false));
    OpParam p;
    Fill(p, HCCL_CMD_ALLGATHER, C(comm), sendBuf, recvBuf, sendCount, dataType, HCCL_REDUCE_RESERVED, 0, stream);
    return Finish(C(comm), p);
}

HcclResult HcclAllGatherV(void* sendBuf, uint64_t sendCount, void* recvBuf, const void* recvCounts, const void* recvDispls,
                          HcclDataType dataType, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(recvCounts);
    CHK_PTR_NULL(recvDispls);
    CommImpl* c = C(comm);
    CHK_RET(CheckDataType("HcclAllGatherV", dataType, false, false));
    OpParam p;
    Fill(p, HCCL_CMD_ALLGATHER_V, c, sendBuf, recvBuf, sendCount, dataType, HCCL_REDUCE_RESERVED, 0, stream);
    ReadU64(recvCounts, (uint32_t)c->nRanks, &p.recvCounts);
    ReadU64(recvDispls, (uint32_t)c->nRanks, &p.rdispls);
    uint64_t total = 0;
    for (int q = 0; q < c->nRanks; ++q) {
        CHK_RET(CheckCount("HcclAllGatherV", p.recvCounts[(size_t)q]));
        CHK_RET(CheckCount("HcclAllGatherV", p.rdispls[(size_t)q] + p.recvCounts[(size_t)q]));
        total += p.recvCounts[(size_t)q];
    }
    if (p.recvCounts[(size_t)c->rank] != sendCount) {
        ReportInputError("EI0003", "HcclAllGatherV", "sendCount", std::to_string(sendCount), "recvCounts[rank]");
        return HCCL_E_PARA;
    }
    if (total == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(recvBuf);
    if (sendCount) CHK_PTR_NULL(sendBuf);
    return Finish(c, p);
}

static HcclResult P2pOne(const char* name, HcclSendRecvType type, void* buf, uint64_t count, HcclDataType dataType, uint32_t peer,
                         HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = C(comm);
    CHK_RET(CheckRank(name, type == HCCL_SEND ? "destRank" : "srcRank", peer, (uint32_t)c->nRanks));
    CHK_RET(CheckCount(name, count));
    CHK_RET(CheckDataType(name, dataType, false, false));
    if (count) CHK_PTR_NULL(buf);
    OpParam p;
    Fill(p, type == HCCL_SEND ? HCCL_CMD_SEND : HCCL_CMD_RECEIVE, c, buf, buf, count, dataType, HCCL_REDUCE_RESERVED, peer, stream);
    HcclSendRecvItem it;
    it.sendRecvType = type; it.buf = buf; it.count = count; it.dataType = dataType; it.remoteRank = peer;
    p.items.push_back(it);
    return Finish(c, p);
}

HcclResult HcclSend(void* sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, HcclComm comm, hcclStream_t stream)
{
    return P2pOne("HcclSend", HCCL_SEND, sendBuf, count, dataType, destRank, comm, stream);
}
HcclResult HcclRecv(void* recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, HcclComm comm, hcclStream_t stream)
{
    return P2pOne("HcclRecv", HCCL_RECV, recvBuf, count, dataType, srcRank, comm, stream);
}

HcclResult HcclBatchSendRecv(HcclSendRecvItem* items, uint32_t itemNum, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = C(comm);
    if (itemNum != 0) CHK_PTR_NULL(items);
    OpParam p;
    Fill(p, HCCL_CMD_BATCH_SEND_RECV, c, nullptr, nullptr, 0, HCCL_DATA_TYPE_INT8, HCCL_REDUCE_RESERVED, 0, stream);
    for (uint32_t i = 0; i < itemNum; ++i) {
        const HcclSendRecvItem& it = items[i];
        if (it.sendRecvType != HCCL_SEND && it.sendRecvType != HCCL_RECV) { ReportInputError("EI0003", "HcclBatchSendRecv", "sendRecvType", std::to_string((int)it.sendRecvType), "HCCL_SEND or HCCL_RECV"); return HCCL_E_PARA; }
        CHK_RET(CheckRank("HcclBatchSendRecv", "remoteRank", it.remoteRank, (uint32_t)c->nRanks));
        CHK_RET(CheckCount("HcclBatchSendRecv", it.count));
        CHK_RET(CheckDataType("HcclBatchSendRecv", it.dataType, false, false));
        if (it.count) CHK_PTR_NULL(it.buf);
        p.items.push_back(it);
    }
    // an empty batch is legal for emulated and host ranks, where every rank must take part in the launch
    if (itemNum == 0 && !c->emulated() && !c->hostComm) return HCCL_SUCCESS;
    return Finish(c, p);
}

HcclResult HcclAlltoAllV(const void* sendBuf, const void* sendCounts, const void* sdispls, HcclDataType sendType, const void* recvBuf,
                         const void* recvCounts, const void* rdispls, HcclDataType recvType, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(sendCounts); CHK_PTR_NULL(sdispls); CHK_PTR_NULL(recvCounts); CHK_PTR_NULL(rdispls);
    CommImpl* c = C(comm);
    CHK_RET(CheckDataType("HcclAlltoAllV", sendType, false, false));
    CHK_RET(CheckDataType("HcclAlltoAllV", recvType, false, false));
    if (DataTypeSize(sendType) != DataTypeSize(recvType)) { ReportInputError("EI0003", "HcclAlltoAllV", "recvType", DataTypeName(recvType), "a type of the same size as sendType"); return HCCL_E_PARA; }
    OpParam p;
    Fill(p, HCCL_CMD_ALLTOALLV, c, sendBuf, const_cast<void*>(recvBuf), 0, sendType, HCCL_REDUCE_RESERVED, 0, stream);
    p.recvType = recvType;
    const uint32_t n = (uint32_t)c->nRanks;
    ReadU64(sendCounts, n, &p.sendCounts); ReadU64(sdispls, n, &p.sdispls); ReadU64(recvCounts, n, &p.recvCounts); ReadU64(rdispls, n, &p.rdispls);
    uint64_t maxCount = 0, sendTotal = 0, recvTotal = 0;
    for (uint32_t q = 0; q < n; ++q) {
        maxCount = std::max(maxCount, std::max(p.sendCounts[q], p.recvCounts[q]));
        sendTotal += p.sendCounts[q];
        recvTotal += p.recvCounts[q];
    }
    CHK_RET(CheckCount("HcclAlltoAllV", maxCount));
    p.count = maxCount;
    if (sendTotal) CHK_PTR_NULL(sendBuf);
    if (recvTotal) CHK_PTR_NULL(recvBuf);
    return Finish(c, p);
}

HcclResult HcclAlltoAll(const void* sendBuf, uint64_t sendCount, HcclDataType sendType, const void* recvBuf, uint64_t recvCount,
                        HcclDataType recvType, HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = C(comm);
    if (sendCount == 0 && recvCount == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(sendBuf);
    CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckDataType("HcclAlltoAll", sendType, false, false));
    CHK_RET(CheckDataType("HcclAlltoAll", recvType, false, false));
    if (sendCount != recvCount || DataTypeSize(sendType) != DataTypeSize(recvType)) {
        ReportInputError("EI0003", "HcclAlltoAll", "recvCount", std::to_string(recvCount), "sendCount, with types of equal size");
        return HCCL_E_PARA;
    }
    CHK_RET(CheckCount("HcclAlltoAll", sendCount * (uint64_t)c->nRanks));
    OpParam p;
    Fill(p, HCCL_CMD_ALLTOALL, c, sendBuf, const_cast<void*>(recvBuf), sendCount, sendType, HCCL_REDUCE_RESERVED, 0, stream);
    p.recvType = recvType;
    for (int q = 0; q < c->nRanks; ++q) {
        p.sendCounts.push_back(sendCount); p.sdispls.push_back(sendCount * (uint64_t)q);
        p.recvCounts.push_back(recvCount); p.rdispls.push_back(recvCount * (uint64_t)q);
    }
    p.globalMaxBytes = sendCount * DataTypeSize(sendType);
    return Finish(c, p);
}

HcclResult HcclAlltoAllVC(const void* sendBuf, const void* sendCountMatrix, HcclDataType sendType, const void* recvBuf, HcclDataType recvType,
                          HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CHK_PTR_NULL(sendCountMatrix);
    CommImpl* c = C(comm);
    CHK_RET(CheckDataType("HcclAlltoAllVC", sendType, false, false));
    CHK_RET(CheckDataType("HcclAlltoAllVC", recvType, false, false));
    if (DataTypeSize(sendType) != DataTypeSize(recvType)) return HCCL_E_PARA;
    const uint32_t n = (uint32_t)c->nRanks, me = (uint32_t)c->rank;
    const uint64_t* m = static_cast<const uint64_t*>(sendCountMatrix);
    OpParam p;
    Fill(p, HCCL_CMD_ALLTOALLVC, c, sendBuf, const_cast<void*>(recvBuf), 0, sendType, HCCL_REDUCE_RESERVED, 0, stream);
    p.recvType = recvType;
    // row `me` = what this rank sends; column `me` = what it receives; displacements are the running sums
    uint64_t sd = 0, rd = 0, maxCount = 0, total = 0;
    for (uint32_t q = 0; q < n; ++q) {
        const uint64_t s = m[(size_t)me * n + q], r = m[(size_t)q * n + me];
        p.sendCounts.push_back(s); p.sdispls.push_back(sd); sd += s;
        p.recvCounts.push_back(r); p.rdispls.push_back(rd); rd += r;
    }
    for (size_t i = 0; i < (size_t)n * n; ++i) { maxCount = std::max(maxCount, m[i]); total += m[i]; }
    CHK_RET(CheckCount("HcclAlltoAllVC", maxCount));
    if (total == 0) return HCCL_SUCCESS;
    if (sd) CHK_PTR_NULL(sendBuf);
    if (rd) CHK_PTR_NULL(recvBuf);
    p.count = maxCount;
    p.globalMaxBytes = maxCount * DataTypeSize(sendType);
    return Finish(c, p);
}

HcclResult HcclReduce(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, HcclComm comm,
                      hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    if (count == 0) return HCCL_SUCCESS;
    CommImpl* c = C(comm);
    CHK_PTR_NULL(sendBuf);
    CHK_RET(CheckRank("HcclReduce", "root", root, (uint32_t)c->nRanks));
    if ((uint32_t)c->rank == root) CHK_PTR_NULL(recvBuf);
    CHK_RET(CheckCount("HcclReduce", count));
    CHK_RET(CheckDataType("HcclReduce", dataType, true, false));
    CHK_RET(CheckReduceOp("HcclReduce", dataType, op));
    OpParam p;
    Fill(p, HCCL_CMD_REDUCE, c, sendBuf, (uint32_t)c->rank == root ? recvBuf : nullptr, count, dataType, op, root, stream);
    return Finish(c, p);
}

HcclResult HcclBarrier(HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    OpParam p;
    Fill(p, HCCL_CMD_BARRIER, C(comm), nullptr, nullptr, 0, HCCL_DATA_TYPE_INT8, HCCL_REDUCE_RESERVED, 0, stream);
    return Finish(C(comm), p);
}

// ---------------------------------------------------------------- graph-mode twins (hccl_graph_mode.h)
namespace {
thread_local std::map<std::string, CommImpl*> g_boundComms;

HcclResult ResolveGroup(const char* group, CommImpl** out)
{
    CHK_PTR_NULL(group);
    auto bound = g_boundComms.find(group);
    const std::vector<CommImpl*> all = GroupFind(group);
    if (bound != g_boundComms.end() && std::find(all.begin(), all.end(), bound->second) != all.end()) { *out = bound->second; return HCCL_SUCCESS; }
    if (all.empty()) { HCCL_ERROR("no communicator named '%s' in this process", group); return HCCL_E_NOT_FOUND; }
    if (all.size() == 1) { *out = all[0]; return HCCL_SUCCESS; }
    // several ranks of the group live in this process: take the one on the current GPU if that settles it
    int dev = -1;
    CommImpl* onDev = nullptr;
    int matches = 0;
    if (cudaGetDevice(&dev) == cudaSuccess)
        for (CommImpl* c : all)
            if (!c->hostComm && !c->emulated() && c->device == dev) { onDev = c; ++matches; }
    (void)cudaGetLastError();
    if (matches == 1) { *out = onDev; return HCCL_SUCCESS; }
    HCCL_ERROR("group '%s' has %zu communicators in this process: bind one to the calling thread with HcclGroupBindThread", group, all.size());
    return HCCL_E_PARA;
}

// A node's resource pack: nothing in it is needed, but a pack that cannot be right is reported.
HcclResult CheckResPack(const HcclResPackGraphMode* res)
{
    if (!res) return HCCL_SUCCESS;
    if (res->size != sizeof(HcclResPackGraphMode)) { HCCL_ERROR("HcclResPackGraphMode.size is %u, expected %zu", res->size, sizeof(HcclResPackGraphMode)); return HCCL_E_PARA; }
    if ((res->scratchBytes && !res->scratch) || (res->slaveStreamNum && !res->slaveStreams)) return HCCL_E_PTR;
    return HCCL_SUCCESS;
}

struct GraphNode {
    CommImpl* comm = nullptr;
    HcclResult Begin(const char* group, const char* tag, const HcclResPackGraphMode* res)
    {
        CHK_RET(ResolveGroup(group, &comm));
        CHK_RET(CheckResPack(res));
        g_graphTag = (tag && *tag) ? tag : nullptr;
        return HCCL_SUCCESS;
    }
    ~GraphNode() { g_graphTag = nullptr; }
};
}  // namespace

HcclResult HcclGroupGetComm(const char* group, HcclComm* comm)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    *comm = c;
    return HCCL_SUCCESS;
}
HcclResult HcclGroupBindThread(HcclComm comm)
{
    CHK_PTR_NULL(comm);
    g_boundComms[C(comm)->name] = C(comm);
    return HCCL_SUCCESS;
}
HcclResult HcclGroupUnbindThread(const char* group)
{
    CHK_PTR_NULL(group);
    g_boundComms.erase(group);
    return HCCL_SUCCESS;
}
HcclResult HcclCalcOpResGraphMode(const char* group, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp, HcclOpResource* res)
{
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    return HcclCalcOpResource(c, op, count, dataType, reduceOp, 0, res);
}

HcclResult HcclCalcOpResOnlineGraphMode(const char* group, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp, int registered,
                                        HcclOpResource* res)
{
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    return HcclCalcOpResource(c, op, count, dataType, reduceOp, registered, res);
}

struct HcclOpParamGraphMode {
    HcclCMDType op = HCCL_CMD_ALLREDUCE;
    uint64_t count = 0, bufferBytes = 0;
    uint32_t rankSize = 8, blockLimit = 0;
    HcclDataType dataType = HCCL_DATA_TYPE_FP32;
    HcclReduceOp reduceOp = HCCL_REDUCE_SUM;
    int registered = 0, switchReduces = 1;
};
HcclResult HcclCreateOpParamGraphMode(HcclOpParamGraphMode** opParam)
{
    CHK_PTR_NULL(opParam);
    *opParam = new (std::nothrow) HcclOpParamGraphMode();
    return *opParam ? HCCL_SUCCESS : HCCL_E_MEMORY;
}
HcclResult HcclDestroyOpParamGraphMode(HcclOpParamGraphMode* opParam)
{
    CHK_PTR_NULL(opParam);
    delete opParam;
    return HCCL_SUCCESS;
}
HcclResult HcclSetOpParamGraphModeOpType(HcclOpParamGraphMode* opParam, const char* opType)
{
    CHK_PTR_NULL(opParam); CHK_PTR_NULL(opType);
    std::string s;
    for (const char* p = opType; *p; ++p)
        if (*p != '_') s.push_back((char)tolower((unsigned char)*p));
    if (s.compare(0, 4, "hcom") == 0) s.erase(0, 4);
    else if (s.compare(0, 4, "hccl") == 0) s.erase(0, 4);
    for (int op = 0; op < (int)HCCL_CMD_MAX; ++op) {
        std::string n;
        for (const char* p = CmdName((HcclCMDType)op); p && *p; ++p) n.push_back((char)tolower((unsigned char)*p));
        if (!n.empty() && n == s) { opParam->op = (HcclCMDType)op; return HCCL_SUCCESS; }
    }
    HCCL_ERROR("HcclSetOpParamGraphModeOpType: unknown operator '%s'", opType);
    return HCCL_E_PARA;
}
HcclResult HcclSetOpParamGraphModeDataCount(HcclOpParamGraphMode* opParam, uint64_t dataCount) { CHK_PTR_NULL(opParam); opParam->count = dataCount; return HCCL_SUCCESS; }
HcclResult HcclSetOpParamGraphModeRankSize(HcclOpParamGraphMode* opParam, uint32_t rankSize)
{
    CHK_PTR_NULL(opParam);
    if (rankSize < 1 || rankSize > (uint32_t)kMaxDevRanks) return HCCL_E_PARA;
    opParam->rankSize = rankSize;
    return HCCL_SUCCESS;
}
HcclResult HcclSetOpParamGraphModeHCCLBufferSize(HcclOpParamGraphMode* opParam, uint64_t bufferBytes) { CHK_PTR_NULL(opParam); opParam->bufferBytes = bufferBytes; return HCCL_SUCCESS; }
HcclResult HcclSetOpParamGraphModeDataType(HcclOpParamGraphMode* opParam, HcclDataType dataType)
{
    CHK_PTR_NULL(opParam);
    if (DataTypeSize(dataType) == 0) return HCCL_E_PARA;
    opParam->dataType = dataType;
    return HCCL_SUCCESS;
}
HcclResult HcclSetOpParamGraphModeReduceType(HcclOpParamGraphMode* opParam, HcclReduceOp reduceOp) { CHK_PTR_NULL(opParam); opParam->reduceOp = reduceOp; return HCCL_SUCCESS; }
HcclResult HcclSetOpParamGraphModeRegistered(HcclOpParamGraphMode* opParam, int registered, int switchReduces)
{
    CHK_PTR_NULL(opParam);
    opParam->registered = registered != 0;
    opParam->switchReduces = switchReduces != 0;
    return HCCL_SUCCESS;
}
HcclResult HcclSetOpParamGraphModeBlockLimit(HcclOpParamGraphMode* opParam, uint32_t blockLimit)
{
    CHK_PTR_NULL(opParam);
    if (blockLimit > (uint32_t)kMaxBlocks) return HCCL_E_PARA;
    opParam->blockLimit = blockLimit;
    return HCCL_SUCCESS;
}
HcclResult HcclCalcOpResOpParamGraphMode(const HcclOpParamGraphMode* opParam, uint64_t* opMemSize, uint32_t* streamNum, uint32_t* taskNum, uint32_t* blockNum,
                                         char algName[128])
{
    CHK_PTR_NULL(opParam);
    HcclOpResource r;
    CHK_RET(HcclCalcOpResOfflineGraphMode(opParam->rankSize, opParam->switchReduces, opParam->bufferBytes, opParam->op, opParam->count, opParam->dataType,
                                          opParam->reduceOp, opParam->registered, &r));
    if (opMemSize) *opMemSize = r.scratchBytes;
    if (streamNum) *streamNum = r.streams;
    if (taskNum) *taskNum = r.launches;
    if (blockNum) *blockNum = opParam->blockLimit && r.blocks > opParam->blockLimit ? opParam->blockLimit : r.blocks;
    if (algName) snprintf(algName, 128, "%s", r.algName);
    return HCCL_SUCCESS;
}
HcclResult HcclSelectAlgGraphMode(const char* group, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType, uint32_t blockLimit,
                                  bool* onDevice, char algName[128])
{
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    (void)blockLimit;                       // the grid does not change which algorithm runs
    HcclOpResource r;
    CHK_RET(HcclCalcOpResource(c, opType, count, dataType, op, 0, &r));
    if (onDevice) *onDevice = r.engine != (uint32_t)HCCL_ENGINE_HOSTCPU;
    if (algName) snprintf(algName, 128, "%s", r.algName);
    return HCCL_SUCCESS;
}
HcclResult HcclCalcBlockNumGraphMode(const char* group, uint64_t count, HcclDataType dataType, HcclReduceOp op, HcclCMDType opType, uint32_t blockLimit,
                                     uint32_t* numBlocks)
{
    CHK_PTR_NULL(numBlocks);
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    HcclOpResource r;
    CHK_RET(HcclCalcOpResource(c, opType, count, dataType, op, 0, &r));
    *numBlocks = blockLimit && r.blocks > blockLimit ? blockLimit : r.blocks;
    return HCCL_SUCCESS;
}
HcclResult HcclGetAlgExecParamGraphMode(const char* tag, const char* group, uint64_t count, HcclCMDType opType, HcclDataType dataType, HcclReduceOp op,
                                        void** commContext, uint64_t* len)
{
    CHK_PTR_NULL(commContext); CHK_PTR_NULL(len);
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    void* args = nullptr;
    CHK_RET(HcclKfcAllocOpArgs(&args));
    HcclKfcOpArgsSetSrcDataType(args, (uint8_t)dataType);
    HcclKfcOpArgsSetDstDataType(args, (uint8_t)dataType);
    HcclKfcOpArgsSetReduceType(args, (uint32_t)op);
    HcclKfcOpArgsSetCount(args, count);
    const HcclResult r = HcclCreateOpResCtx(c, (uint8_t)opType, args, commContext);
    HcclKfcFreeOpArgs(args);
    if (r != HCCL_SUCCESS) return r;
    *len = sizeof(HcclMc2ResCtx);
    HCCL_INFO("graph node %s: communicator context of group %s for %s", tag ? tag : "(untagged)", group, CmdName(opType));
    return HCCL_SUCCESS;
}
HcclResult HcclSetBlockLimitGraphMode(const char* group, uint32_t blockLimit)
{
    CommImpl* c = nullptr;
    CHK_RET(ResolveGroup(group, &c));
    if (blockLimit > (uint32_t)kMaxBlocks) return HCCL_E_PARA;
    std::lock_guard<std::mutex> lk(c->opMu);
    c->cfg.maxBlocks = blockLimit;
    if (c->plans) c->plans->Clear();        // launch shapes were planned for the old grid
    return HCCL_SUCCESS;
}

#define GRAPH_NODE() GraphNode node; CHK_RET(node.Begin(group, tag, res))
HcclResult HcclAllReduceGraphMode(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, const char* group,
                                  const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAllReduce(sendBuf, recvBuf, count, dataType, op, node.comm, stream);
}
HcclResult HcclBroadcastGraphMode(void* buf, uint64_t count, HcclDataType dataType, uint32_t root, const char* group, const char* tag,
                                  const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclBroadcast(buf, count, dataType, root, node.comm, stream);
}
HcclResult HcclReduceScatterGraphMode(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, HcclReduceOp op, const char* group,
                                      const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclReduceScatter(sendBuf, recvBuf, recvCount, dataType, op, node.comm, stream);
}
HcclResult HcclAllGatherGraphMode(void* sendBuf, void* recvBuf, uint64_t sendCount, HcclDataType dataType, const char* group, const char* tag,
                                  const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAllGather(sendBuf, recvBuf, sendCount, dataType, node.comm, stream);
}
HcclResult HcclReduceGraphMode(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType dataType, HcclReduceOp op, uint32_t root, const char* group,
                               const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclReduce(sendBuf, recvBuf, count, dataType, op, root, node.comm, stream);
}
HcclResult HcclScatterGraphMode(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType dataType, uint32_t root, const char* group,
                                const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclScatter(sendBuf, recvBuf, recvCount, dataType, root, node.comm, stream);
}
HcclResult HcclAlltoAllGraphMode(const void* sendBuf, uint64_t sendCount, HcclDataType sendType, const void* recvBuf, uint64_t recvCount,
                                 HcclDataType recvType, const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAlltoAll(sendBuf, sendCount, sendType, recvBuf, recvCount, recvType, node.comm, stream);
}
HcclResult HcclAllGatherVGraphMode(void* sendBuf, void* recvBuf, uint64_t sendCount, const void* recvCounts, const void* recvDispls, HcclDataType dataType,
                                   const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAllGatherV(sendBuf, sendCount, recvBuf, recvCounts, recvDispls, dataType, node.comm, stream);
}
HcclResult HcclReduceScatterVGraphMode(void* sendBuf, const void* sendCounts, const void* sendDispls, void* recvBuf, uint64_t recvCount, HcclDataType dataType,
                                       HcclReduceOp op, const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclReduceScatterV(sendBuf, sendCounts, sendDispls, recvBuf, recvCount, dataType, op, node.comm, stream);
}
HcclResult HcclAlltoAllVGraphMode(const void* sendBuf, const void* sendCounts, const void* sdispls, HcclDataType sendType, const void* recvBuf,
                                  const void* recvCounts, const void* rdispls, HcclDataType recvType, const char* group, const char* tag,
                                  const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAlltoAllV(sendBuf, sendCounts, sdispls, sendType, recvBuf, recvCounts, rdispls, recvType, node.comm, stream);
}
HcclResult HcclAlltoAllVCGraphMode(const void* sendBuf, const void* sendCountMatrix, HcclDataType sendType, const void* recvBuf, HcclDataType recvType,
                                   const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclAlltoAllVC(sendBuf, sendCountMatrix, sendType, recvBuf, recvType, node.comm, stream);
}
HcclResult HcclSendGraphMode(void* sendBuf, uint64_t count, HcclDataType dataType, uint32_t destRank, const char* group, const char* tag,
                             const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclSend(sendBuf, count, dataType, destRank, node.comm, stream);
}
HcclResult HcclRecvGraphMode(void* recvBuf, uint64_t count, HcclDataType dataType, uint32_t srcRank, const char* group, const char* tag,
                             const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclRecv(recvBuf, count, dataType, srcRank, node.comm, stream);
}
HcclResult HcclBarrierGraphMode(const char* group, const char* tag, const HcclResPackGraphMode* res, hcclStream_t stream)
{
    GRAPH_NODE();
    return HcclBarrier(node.comm, stream);
}
#undef GRAPH_NODE

}  // extern "C"
