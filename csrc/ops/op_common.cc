// Operator orchestration: parameter model -> selection -> sole executor (chunk
// loop over the staging slab) -> kernel launch.
//
// Reference flow (src/ops/op_common/op_common.cc): Selector() :184 (status gate,
// topology cache, cost model / cost table, tuner) -> HcclExecOp() :1259
// (resource context by algTag, first-call consistency check :1898-1936, engine
// dispatch, profiling report :1440), with the single-rank shortcut
// SingleRankProc :4458 and the fast paths that skip selection for a repeated
// call signature (op_common.cc:432, :677).  The chunk loop bound follows
// ins_v2_all_reduce_sole_executor.cc:240-266: bytes per loop =
// floor(region / scratchMultiple / 128) * 128, last loop takes the remainder.
#include "op_common.h"
#include <algorithm>
#include <chrono>
#include <cstring>
#include <sstream>
#include "../core/algo_plugin.h"
#include "../core/log.h"
#include "../core/plan_cache.h"
#include "../cpu/host_comm.h"
#include "../kernels/dev_types.h"
#include "param_check.h"
#include "profiling.h"

namespace hccl {

namespace {

bool Aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0; }
uint64_t AlignDown(uint64_t v, uint64_t a) { return v / a * a; }
uint64_t AlignUp(uint64_t v, uint64_t a) { return (v + a - 1) / a * a; }

int BlocksFor(const CommImpl* c, uint64_t bytesPerRank, DevAlg alg)
{
    const int maxB = c->MaxBlocks();
    if (alg == DALG_AR_LL || alg == DALG_AG_LL || alg == DALG_RS_LL || alg == DALG_BCAST_LL || alg == DALG_A2A_LL) {
        int nb = (int)((bytesPerRank + 4095) / 4096);   // 512 threads x 8 payload bytes: one line per thread while blocks last
        return std::max(1, std::min(nb, maxB));
    }
    // one block per 16 KiB of traffic, at least 1, at most the configured ceiling: remote loads need many bytes in
    // flight (about 2.5 MB per direction to fill an NVLink 5 port), and a block that walks a long range alone pays one
    // NVLink round trip per pass
    uint64_t nb = (bytesPerRank + (16u << 10) - 1) / (16u << 10);
    return (int)std::max<uint64_t>(1, std::min<uint64_t>(nb, (uint64_t)maxB));
}

struct RegInfo {
    bool reg = false;
    const char* peer[kMaxDevRanks] = {nullptr};
    const char* mc = nullptr;
};
RegInfo Reg(const CommImpl* c, const void* p, uint64_t bytes)
{
    RegInfo r;
    if (p != nullptr && bytes > 0) r.reg = c->Lookup(p, bytes, r.peer, &r.mc);
    return r;
}

// First call of each operator type: all ranks compare what they were called with (reference inconsistent_check.h:
// op type, data type, count, root, buffer size), so a mismatched call fails with a message instead of hanging.
struct ConsistencyRecord { uint32_t op, dtype, redOp, root; uint64_t count, bufferBytes; };
HcclResult FirstCallCheck(CommImpl* c, const OpParam& p)
{
    if (!c->bs || c->firstOpChecked[p.op] || !GetEnvConfig().dfs.inconsistentCheck) return HCCL_SUCCESS;
    c->firstOpChecked[p.op] = true;
    const bool countMustMatch = p.op != HCCL_CMD_ALLTOALLV && p.op != HCCL_CMD_SEND && p.op != HCCL_CMD_RECEIVE &&
                                p.op != HCCL_CMD_BATCH_SEND_RECV && p.op != HCCL_CMD_ALLGATHER_V && p.op != HCCL_CMD_REDUCE_SCATTER_V;
    if (p.op == HCCL_CMD_SEND || p.op == HCCL_CMD_RECEIVE || p.op == HCCL_CMD_BATCH_SEND_RECV) return HCCL_SUCCESS;  // not collective
    ConsistencyRecord mine = {(uint32_t)p.op, (uint32_t)p.dtype, (uint32_t)p.redOp, p.root, countMustMatch ? p.count : 0, c->cfg.bufferBytes};
    std::vector<ConsistencyRecord> all((size_t)c->nRanks);
    CHK_RET(c->bs->AllGather(&mine, all.data(), sizeof(mine)));
    for (int r = 0; r < c->nRanks; ++r) {
        if (memcmp(&all[(size_t)r], &mine, sizeof(mine)) != 0) {
            HCCL_ERROR("comm %s: rank %d and rank %d called %s with different parameters (dtype %u/%u, op %u/%u, root %u/%u, count %llu/%llu, buffer %llu/%llu)",
                       c->name.c_str(), c->rank, r, CmdName(p.op), mine.dtype, all[(size_t)r].dtype, mine.redOp, all[(size_t)r].redOp, mine.root,
                       all[(size_t)r].root, (unsigned long long)mine.count, (unsigned long long)all[(size_t)r].count,
                       (unsigned long long)mine.bufferBytes, (unsigned long long)all[(size_t)r].bufferBytes);
            return HCCL_E_PARA;
        }
    }
    return HCCL_SUCCESS;
}

HcclResult LocalCopy(void* dst, const void* src, uint64_t bytes, cudaStream_t s)
{
    if (bytes == 0 || dst == src) return HCCL_SUCCESS;
    CHK_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, s));
    return HCCL_SUCCESS;
}

// Single-rank communicator: every collective degenerates to a local copy (reference SingleRankProc op_common.cc:4458).
HcclResult SingleRank(CommImpl*, const OpParam& p)
{
    const uint64_t es = DataTypeSize(p.dtype);
    switch (p.op) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE: case HCCL_CMD_ALLGATHER: case HCCL_CMD_REDUCE_SCATTER:
        case HCCL_CMD_SCATTER: case HCCL_CMD_ALLTOALL:
            return LocalCopy(p.recv, p.send, p.count * es, p.stream);
        case HCCL_CMD_ALLGATHER_V:
            return LocalCopy((char*)p.recv + p.rdispls[0] * es, p.send, p.count * es, p.stream);
        case HCCL_CMD_REDUCE_SCATTER_V:
            return LocalCopy(p.recv, (const char*)p.send + p.sdispls[0] * es, p.count * es, p.stream);
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
            return LocalCopy((char*)p.recv + p.rdispls[0] * DataTypeSize(p.recvType), (const char*)p.send + p.sdispls[0] * es, p.sendCounts[0] * es, p.stream);
        default: return HCCL_SUCCESS;  // broadcast, barrier
    }
}

struct Exec {
    CommImpl* c;
    const OpParam& p;
    const OpDesc& d;          // buffer facts every rank agrees on: whatever a peer can observe (where it reads this rank's data,
                              // how many launches and blocks an operator takes) is derived from these, never from local lookups alone
    const AlgEntry* alg;
    DevAlg dalg;
    uint64_t es;
    int P, me;
    LaunchTarget tgt;
    const StageLayout& L;
    Exec(CommImpl* comm, const OpParam& param, const OpDesc& desc, const AlgEntry* a)
        : c(comm), p(param), d(desc), alg(a), dalg((DevAlg)a->devAlg), es(DataTypeSize(param.dtype)), P(comm->nRanks), me(comm->rank),
          tgt(comm->Target(param.stream)), L(comm->layout()) {}

    void FillStageIn(CollArgs& a) const { for (int q = 0; q < P; ++q) a.src[q] = c->StageBase(q) + L.inOff; a.srcMc = c->StageMcBase() ? c->StageMcBase() + L.inOff : nullptr; }
    void FillXch(CollArgs& a) const { for (int q = 0; q < P; ++q) a.xch[q] = c->StageBase(q) + L.xchOff; }
    HcclResult Launch(const CollArgs& a, uint64_t trafficBytes) const
    {
        if (p.castScale) return LaunchCollectiveExt(tgt, dalg, p.dtype, p.outType, a, BlocksFor(c, trafficBytes, dalg));
        return LaunchCollective(tgt, dalg, p.dtype, a, BlocksFor(c, trafficBytes, dalg));
    }
    uint64_t esOut() const { return p.castScale ? DataTypeSize(p.outType) : es; }
    uint64_t LoopBytes(uint64_t region, uint64_t multiple) const { return AlignDown(region / multiple, 128); }
    // The push forms land data in the receivers' stage-in region, which holds two landing copies taken in turn; the
    // second starts at the same offset for every operator, whatever its size, so that copies of different operators
    // never overlap.
    uint64_t LandingCopyBytes() const { return AlignDown(L.inBytes / 2, 128); }

    // ---- AllReduce / Reduce --------------------------------------------------
    HcclResult AllReduceLike() const
    {
        const uint64_t total = p.count * es;
        const bool isReduce = p.op == HCCL_CMD_REDUCE;
        const bool ll = dalg == DALG_AR_LL;
        if (dalg == DALG_AR_PUSH_TWOSHOT) {
            // slices pushed into their owners' landing copies (p slots of one slice each), reduced slices exchanged
            // through the exchange region: the input is read once and never staged
            const uint64_t landing = LandingCopyBytes();
            if (landing < 256ull * (uint64_t)P) return HCCL_E_MEMORY;
            const uint64_t limit = std::min(AlignDown(landing - 16ull * (uint64_t)P, 128), LoopBytes(L.xchBytes, 1));
            if (limit == 0) return HCCL_E_MEMORY;
            for (uint64_t off = 0; off < total; off += limit) {
                const uint64_t n = std::min(limit, total - off);
                CollArgs a;
                memset(&a, 0, sizeof(a));
                a.in = (const char*)p.send + off;
                a.out = (char*)p.recv + off;
                a.bytes = n;
                a.op = (int)p.redOp;
                a.chunk = landing;
                FillStageIn(a);
                FillXch(a);
                CHK_RET(Launch(a, n / (uint64_t)P * 2 + 1));
            }
            return HCCL_SUCCESS;
        }
        RegInfo in = Reg(c, p.send, total), out = Reg(c, p.recv, total);
        const bool inDirect = d.inRegistered && d.aligned16 && in.reg && Aligned16(p.send);
        const bool nvlsAlg = dalg == DALG_AR_NVLS;
        // NVLS needs a multicast alias for its source; a registered buffer without one is staged.  One-shot in place on
        // a registered buffer would let a rank overwrite its input with sums while its peers still read it (every rank
        // reads the whole message of every peer between the two barriers): that case is staged as well.
        const bool oneShotForm = dalg == DALG_AR_ONESHOT || dalg == DALG_AR_ONESHOT_CAST;
        const bool readsInputLate = oneShotForm || dalg == DALG_AR_RHD;      // a peer may read this rank's input after this rank wrote output
        const bool useInDirect = inDirect && (!nvlsAlg || (d.inMulticast && in.mc != nullptr)) && !ll && !(readsInputLate && d.inPlace);
        const bool outAligned = Aligned16(p.recv);
        const bool pushOut = (dalg == DALG_AR_TWOSHOT || nvlsAlg) && d.outRegistered && d.aligned16 && out.reg && outAligned &&
                             (!nvlsAlg || (d.outMulticast && out.mc != nullptr)) && !isReduce;
        uint64_t chunk = total;
        if (!ll) {
            uint64_t limit = ~0ull;
            if (!useInDirect) limit = std::min(limit, LoopBytes(L.inBytes, 1));
            const bool needXch = (dalg == DALG_AR_TWOSHOT && !pushOut) || (nvlsAlg && !pushOut) || dalg == DALG_REDUCE_TWOSHOT ||
                                 dalg == DALG_AR_TWOSHOT_CAST || dalg == DALG_AR_RHD;
            // the cast form keeps output elements in the exchange region: count the limit in input bytes
            if (needXch) limit = std::min(limit, LoopBytes(L.xchBytes * es / std::max<uint64_t>(es, esOut()), 1));
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min(total, limit);
        }
        for (uint64_t off = 0; off < total; off += chunk) {
            const uint64_t n = std::min(chunk, total - off);
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send + off;
            a.out = (char*)p.recv + off / es * esOut();
            a.bytes = n;
            a.op = (int)p.redOp;
            a.root = (int)p.root;
            a.scale = p.castScale ? p.scale : 1.0f;
            if (useInDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q] + off; a.srcMc = in.mc ? in.mc + off : nullptr; }
            else { FillStageIn(a); a.mode |= MODE_STAGE_IN; }
            FillXch(a);
            if (pushOut) {
                a.mode |= MODE_PUSH;
                for (int q = 0; q < P; ++q) a.dst[q] = const_cast<char*>(out.peer[q]) + off;
                a.dstMc = out.mc ? const_cast<char*>(out.mc) + off : nullptr;
            } else if (nvlsAlg) {
                a.mode |= MODE_STAGE_OUT;
                for (int q = 0; q < P; ++q) a.dst[q] = a.xch[q];
                a.dstMc = c->StageMcBase() + L.xchOff;
            } else if (!outAligned) {
                a.mode |= MODE_STAGE_OUT;
            }
            if (dalg == DALG_REDUCE_ONESHOT) a.mode |= MODE_PUSH;   // one-shot flavour of ReduceBody
            CHK_RET(Launch(a, oneShotForm || dalg == DALG_REDUCE_ONESHOT ? n : n / (uint64_t)P * 2 + 1));
        }
        return HCCL_SUCCESS;
    }

    // ---- ReduceScatter(V) ----------------------------------------------------
    HcclResult ReduceScatterLike() const
    {
        const bool v = p.op == HCCL_CMD_REDUCE_SCATTER_V;
        uint64_t cntB[kMaxDevRanks], dspB[kMaxDevRanks], maxCnt = 0, inSpan = 0;
        for (int q = 0; q < P; ++q) {
            cntB[q] = (v ? p.sendCounts[(size_t)q] : p.count) * es;
            dspB[q] = (v ? p.sdispls[(size_t)q] : p.count * (uint64_t)q) * es;
            maxCnt = std::max(maxCnt, cntB[q]);
            inSpan = std::max(inSpan, dspB[q] + cntB[q]);
        }
        if (dalg == DALG_RS_PUSH) {
            // block q pushed into rank q's landing copy (p slots of one chunk each): the input is read once, never staged
            const uint64_t landing = LandingCopyBytes();
            const uint64_t limit = AlignDown(landing / (uint64_t)P, 128);
            if (limit == 0) return HCCL_E_MEMORY;
            const uint64_t block = p.count * es;
            for (uint64_t off = 0; off < block; off += limit) {
                CollArgs a;
                memset(&a, 0, sizeof(a));
                a.in = (const char*)p.send;
                a.out = (char*)p.recv + off;
                a.op = (int)p.redOp;
                a.bytes = std::min(limit, block - off);
                a.chunk = landing;
                for (int q = 0; q < P; ++q) { a.cnt[q] = a.bytes; a.dsp2[q] = dspB[q] + off; }
                FillStageIn(a);
                CHK_RET(Launch(a, a.bytes + 1));
            }
            return HCCL_SUCCESS;
        }
        RegInfo in = Reg(c, p.send, inSpan);
        bool inDirect = d.inRegistered && d.aligned16 && in.reg && Aligned16(p.send);
        for (int q = 0; q < P && inDirect; ++q) inDirect = (dspB[q] & 15u) == 0;
        if (dalg == DALG_RS_NVLS && (!d.inMulticast || in.mc == nullptr)) inDirect = false;
        uint64_t chunk = maxCnt;
        if (!inDirect) {
            const uint64_t limit = AlignDown(L.inBytes / (uint64_t)P, 128);
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min<uint64_t>(std::max<uint64_t>(maxCnt, 1), limit);
        }
        if (dalg == DALG_RS_RING) {
            // the partial sums travel through one exchange slot per step
            const uint64_t limit = AlignDown(L.xchBytes / (uint64_t)std::max(1, P - 1), 128);
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min<uint64_t>(std::max<uint64_t>(chunk, 1), limit);
        }
        if (maxCnt == 0) chunk = 1;
        for (uint64_t off = 0; off < std::max<uint64_t>(maxCnt, 1); off += chunk) {
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send;
            a.out = (char*)p.recv + off / es * esOut();
            a.op = (int)p.redOp;
            a.scale = p.castScale ? p.scale : 1.0f;
            FillXch(a);
            uint64_t sum = 0;
            for (int q = 0; q < P; ++q) {
                a.cnt[q] = cntB[q] > off ? std::min(chunk, cntB[q] - off) : 0;
                a.dsp2[q] = dspB[q] + off;
                a.dsp[q] = inDirect ? dspB[q] + off : (uint64_t)q * AlignUp(chunk, 16);
                sum += a.cnt[q];
            }
            a.bytes = dalg == DALG_RS_RING ? a.cnt[me] : sum;          // the ring's slots are one block wide
            if (inDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q]; a.srcMc = in.mc; }
            else { FillStageIn(a); a.mode |= MODE_STAGE_IN; }
            // the grid must be the same on every rank: size it by the largest block, which all ranks know
            uint64_t biggest = 0;
            for (int q = 0; q < P; ++q) biggest = std::max(biggest, a.cnt[q]);
            CHK_RET(Launch(a, biggest + 1));
            if (maxCnt == 0) break;
        }
        return HCCL_SUCCESS;
    }

    // ---- small-message forms of ReduceScatter / Broadcast / AlltoAll: every pair moves `pair` bytes as LL lines ----
    HcclResult LLExchange() const
    {
        CollArgs a;
        memset(&a, 0, sizeof(a));
        a.op = (int)p.redOp;
        uint64_t pair = 0;
        if (p.op == HCCL_CMD_REDUCE_SCATTER) {
            pair = p.count * es;
            a.in = (const char*)p.send;
            a.out = (char*)p.recv;
            for (int q = 0; q < P; ++q) { a.cnt2[q] = a.cnt[q] = pair; a.dsp2[q] = pair * (uint64_t)q; }
            a.cnt2[me] = 0;
        } else if (p.op == HCCL_CMD_BROADCAST) {
            pair = p.count * es;
            a.in = (const char*)p.send;
            a.out = (char*)p.send;
            a.root = (int)p.root;
            if (me == (int)p.root) { for (int q = 0; q < P; ++q) a.cnt2[q] = q == me ? 0 : pair; }
            else a.cnt[p.root] = pair;
        } else {
            pair = p.sendCounts[0] * es;
            a.in = (const char*)p.send;
            a.out = (char*)p.recv;
            for (int q = 0; q < P; ++q) { a.cnt2[q] = a.cnt[q] = pair; a.dsp2[q] = a.dsp[q] = pair * (uint64_t)q; }
            a.cnt2[me] = 0;
        }
        if (pair > kLLMaxPayload) return HCCL_E_INTERNAL;
        a.bytes = pair;
        if (pair == 0) return HCCL_SUCCESS;
        return Launch(a, pair);
    }

    // ---- AllGather(V) ----------------------------------------------------------
    HcclResult AllGatherLike() const
    {
        const bool v = p.op == HCCL_CMD_ALLGATHER_V;
        uint64_t cntB[kMaxDevRanks], dspB[kMaxDevRanks], maxCnt = 0;
        for (int q = 0; q < P; ++q) {
            cntB[q] = (v ? p.recvCounts[(size_t)q] : p.count) * es;
            dspB[q] = (v ? p.rdispls[(size_t)q] : p.count * (uint64_t)q) * es;
            maxCnt = std::max(maxCnt, cntB[q]);
        }
        const uint64_t myBytes = p.count * es;
        RegInfo in = Reg(c, p.send, myBytes);
        const bool ll = dalg == DALG_AG_LL;
        // a peer pulls block q from rank q's input, so "registered" has to hold on every rank: d.inRegistered does
        const bool inDirect = d.inRegistered && in.reg && !ll;
        const bool inPlace = (const char*)p.send == (char*)p.recv + dspB[me];
        const bool nvlsAlg = dalg == DALG_AG_NVLS;
        RegInfo out;
        uint64_t outSpan = 0;
        for (int q = 0; q < P; ++q) outSpan = std::max(outSpan, dspB[q] + cntB[q]);
        if (nvlsAlg) out = Reg(c, p.recv, outSpan);
        bool nvlsDirect = nvlsAlg && d.outRegistered && d.outMulticast && d.aligned16 && out.reg && out.mc != nullptr && Aligned16(p.recv);
        for (int q = 0; q < P && nvlsDirect; ++q) nvlsDirect = (dspB[q] & 15u) == 0;
        uint64_t chunk = std::max<uint64_t>(maxCnt, 1);
        if (!inDirect && !ll && !nvlsAlg) {
            const uint64_t limit = LoopBytes(L.inBytes, 1);
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min(chunk, limit);
        }
        if (dalg == DALG_AG_RING) {
            const uint64_t limit = AlignDown(L.xchBytes / (uint64_t)std::max(1, P - 1), 128);
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min(chunk, limit);
        }
        if (nvlsAlg && !nvlsDirect) {
            const uint64_t limit = AlignDown(L.xchBytes / (uint64_t)P, 128);      // every rank's block lands in the exchange region
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min(chunk, limit);
        }
        for (uint64_t off = 0; off < std::max<uint64_t>(maxCnt, 1); off += chunk) {
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send + off;
            a.out = (char*)p.recv;
            for (int q = 0; q < P; ++q) {
                a.cnt[q] = cntB[q] > off ? std::min(chunk, cntB[q] - off) : 0;
                a.dsp[q] = dspB[q] + off;
                a.dsp2[q] = nvlsDirect ? a.dsp[q] : (uint64_t)q * AlignUp(chunk, 16);
            }
            a.bytes = a.cnt[me];
            FillXch(a);
            if (inPlace) a.mode |= MODE_INPLACE;
            if (nvlsAlg) {
                if (nvlsDirect) {
                    a.mode |= MODE_PUSH;
                    a.dstMc = const_cast<char*>(out.mc);
                    for (int q = 0; q < P; ++q) a.dst[q] = const_cast<char*>(out.peer[q]);
                } else {
                    a.dstMc = c->StageMcBase() + L.xchOff;
                    for (int q = 0; q < P; ++q) a.dst[q] = a.xch[q];
                }
            } else if (inDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q] + off; }
            else if (!ll) { FillStageIn(a); a.mode |= MODE_STAGE_IN; }
            uint64_t traffic = 0;
            for (int q = 0; q < P; ++q) traffic += a.cnt[q];
            CHK_RET(Launch(a, ll ? a.cnt[me] : traffic));
            if (maxCnt == 0) break;
        }
        return HCCL_SUCCESS;
    }

    // ---- Broadcast ---------------------------------------------------------------
    HcclResult Broadcast() const
    {
        const uint64_t total = p.count * es;
        RegInfo in = Reg(c, p.send, total);
        const bool scatterNvls = dalg == DALG_BCAST_SCATTER_NVLS;      // reads the root like the pull forms, writes like the switch form
        const bool nvlsAlg = dalg == DALG_BCAST_NVLS;
        const bool pipe = dalg == DALG_BCAST_PIPE;
        const bool inDirect = d.inRegistered && in.reg && !nvlsAlg;
        uint64_t limit = ~0ull;
        if (!inDirect && !nvlsAlg) limit = std::min(limit, LoopBytes(L.inBytes, 1));
        if (pipe && !inDirect) limit = std::min(limit, LoopBytes(L.xchBytes, 1));      // the owners' pieces wait in the exchange region
        const bool nvlsDirect = (nvlsAlg || scatterNvls) && d.inRegistered && d.inMulticast && d.aligned16 && in.reg && in.mc != nullptr && Aligned16(p.send);
        if (dalg == DALG_BCAST_TWOSHOT || ((nvlsAlg || scatterNvls) && !nvlsDirect)) limit = std::min(limit, LoopBytes(L.xchBytes, 1));
        if (limit == 0) return HCCL_E_MEMORY;
        const uint64_t chunk = std::min(total, limit);
        for (uint64_t off = 0; off < total; off += chunk) {
            const uint64_t n = std::min(chunk, total - off);
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send + off;
            a.out = (char*)p.send + off;
            a.bytes = n;
            a.root = (int)p.root;
            if (inDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q] + off; }
            else if (!nvlsAlg) { FillStageIn(a); a.mode |= MODE_STAGE_IN; }
            FillXch(a);
            if (nvlsAlg || scatterNvls) {
                if (nvlsDirect) {
                    a.mode |= MODE_PUSH;      // the buffer is symmetric with a multicast alias: store straight into it
                    a.dstMc = const_cast<char*>(in.mc) + off;
                    for (int q = 0; q < P; ++q) a.dst[q] = const_cast<char*>(in.peer[q]) + off;
                } else {
                    a.dstMc = c->StageMcBase() + L.xchOff;
                    for (int q = 0; q < P; ++q) a.dst[q] = a.xch[q];
                }
            }
            if (dalg == DALG_BCAST_ONESHOT) a.mode |= MODE_PUSH;
            if (pipe) {
                if (inDirect) { a.mode |= MODE_PUSH; for (int q = 0; q < P; ++q) a.dst[q] = const_cast<char*>(in.peer[q]) + off; }
                // pieces of about 48 KiB per block row and slice, at most 12 steps; the largest sub-range (slice 0, row 0)
                // sizes the piece, so pieces x piece bytes covers every sub-range
                const uint64_t nbRows = (uint64_t)BlocksFor(c, n, dalg);
                const uint64_t slice = (((n + 15) / 16 + (uint64_t)(P - 1) - 1) / (uint64_t)(P - 1)) * 16;
                const uint64_t sub = (((slice + 15) / 16 + nbRows - 1) / nbRows) * 16;
                const uint64_t pieces = std::max<uint64_t>(1, std::min<uint64_t>(12, (sub + (48u << 10) - 1) / (48u << 10)));
                a.cnt2[0] = pieces;
                a.chunk = (((sub + 15) / 16 + pieces - 1) / pieces) * 16;
            }
            CHK_RET(Launch(a, n));
        }
        return HCCL_SUCCESS;
    }

    // ---- Scatter -----------------------------------------------------------------
    HcclResult Scatter() const
    {
        const uint64_t per = p.count * es;      // bytes every rank receives
        // only the root's buffer matters and the other ranks cannot see whether the root registered it, so the root
        // always publishes the blocks through its slab (a local copy at HBM speed)
        RegInfo in;
        const bool inDirect = false;
        uint64_t chunk = std::max<uint64_t>(per, 1);
        if (!inDirect) {
            const uint64_t limit = AlignDown(L.inBytes / (uint64_t)P, 128);
            if (limit == 0) return HCCL_E_MEMORY;
            chunk = std::min(chunk, limit);
        }
        for (uint64_t off = 0; off < std::max<uint64_t>(per, 1); off += chunk) {
            const uint64_t n = per == 0 ? 0 : std::min(chunk, per - off);
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send;
            a.out = (char*)p.recv + off;
            a.bytes = n;
            a.root = (int)p.root;
            for (int q = 0; q < P; ++q) {
                a.dsp2[q] = per * (uint64_t)q + off;
                a.dsp[q] = inDirect ? a.dsp2[q] : (uint64_t)q * AlignUp(chunk, 16);
            }
            if (inDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q]; }
            else { FillStageIn(a); a.mode |= MODE_STAGE_IN; }
            CHK_RET(Launch(a, n));
            if (per == 0) break;
        }
        return HCCL_SUCCESS;
    }

    // ---- AlltoAll / V / VC -----------------------------------------------------
    HcclResult AlltoAllLike() const
    {
        const uint64_t res = DataTypeSize(p.recvType);
        uint64_t sendB[kMaxDevRanks], sdspB[kMaxDevRanks], recvB[kMaxDevRanks], rdspB[kMaxDevRanks];
        uint64_t span = 0, staged = 0;
        for (int q = 0; q < P; ++q) {
            sendB[q] = p.sendCounts[(size_t)q] * es;
            sdspB[q] = p.sdispls[(size_t)q] * es;
            recvB[q] = p.recvCounts[(size_t)q] * res;
            rdspB[q] = p.rdispls[(size_t)q] * res;
            span = std::max(span, sdspB[q] + sendB[q]);
            staged += AlignUp(sendB[q], 16);
        }
        RegInfo in = Reg(c, p.send, span);
        const bool inDirect = d.inRegistered && in.reg;
        // Chunking on the host needs a loop count all ranks agree on.  It is known for the uniform op and for VC (every
        // rank holds the whole matrix, globalMaxBytes); AlltoAllV counts are private to each rank, so a staged AlltoAllV
        // hands the kernel the window size and the kernel derives the number of passes from all ranks' send sizes.
        uint64_t perPeerLimit = ~0ull;
        if (!inDirect) {
            perPeerLimit = AlignDown(L.inBytes / (uint64_t)P, 128);
            if (perPeerLimit == 0) return HCCL_E_MEMORY;
        }
        (void)staged;
        if (dalg == DALG_A2A_PUSH) {
            // every pair's block lands in the receiver's stage-in region, two copies by parity
            const uint64_t pair = sendB[0], slot = AlignUp(pair, 16), copyBytes = slot * (uint64_t)P;
            if (copyBytes > LandingCopyBytes()) return HCCL_E_INTERNAL;
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send;
            a.out = (char*)p.recv;
            a.bytes = pair;
            a.chunk = LandingCopyBytes();
            for (int q = 0; q < P; ++q) { a.dsp2[q] = sdspB[q]; a.dsp[q] = rdspB[q]; }
            FillStageIn(a);
            return Launch(a, pair * (uint64_t)P);
        }
        uint64_t loops = 1, chunk = ~0ull;
        if (!inDirect && p.op != HCCL_CMD_ALLTOALLV && p.globalMaxBytes > perPeerLimit) {
            chunk = perPeerLimit;
            loops = (p.globalMaxBytes + chunk - 1) / chunk;
        }
        for (uint64_t i = 0; i < loops; ++i) {
            const uint64_t off = loops == 1 ? 0 : i * chunk;
            CollArgs a;
            memset(&a, 0, sizeof(a));
            a.in = (const char*)p.send;
            a.out = (char*)p.recv;
            uint64_t traffic = 0;
            for (int q = 0; q < P; ++q) {
                a.cnt2[q] = sendB[q] > off ? std::min(chunk, sendB[q] - off) : 0;
                a.dsp2[q] = sdspB[q] + off;
                a.cnt[q] = recvB[q] > off ? std::min(chunk, recvB[q] - off) : 0;
                a.dsp[q] = rdspB[q] + off;
                traffic += a.cnt[q];
            }
            a.bytes = traffic;
            FillXch(a);
            if (inDirect) { for (int q = 0; q < P; ++q) a.src[q] = in.peer[q]; }
            else { FillStageIn(a); a.mode |= MODE_STAGE_IN; if (p.op == HCCL_CMD_ALLTOALLV) a.chunk = perPeerLimit; }
            // every rank has to launch the same grid.  The uniform op and VC know the global sizes; AlltoAllV does
            // not (counts are private to each rank), so it always runs with the full grid: a large exchange is bound
            // by the bytes in flight, and the extra block rows of a small one only add their own (parallel) barriers.
            if (p.op == HCCL_CMD_ALLTOALLV) CHK_RET(LaunchCollective(tgt, dalg, p.dtype, a, c->MaxBlocks()));
            else CHK_RET(Launch(a, std::min(chunk, p.globalMaxBytes) * (uint64_t)P));
        }
        return HCCL_SUCCESS;
    }

    // ---- Send / Recv / BatchSendRecv -----------------------------------------
    HcclResult PointToPoint() const
    {
        // two items towards the same peer in the same direction share one sequence counter: they go in separate launches
        std::vector<HcclSendRecvItem> rest(p.items);
        while (!rest.empty() || p.items.empty()) {
            P2pArgs a;
            memset(&a, 0, sizeof(a));
            a.halfBytes = L.mailboxHalf;
            a.mailboxOff = L.mailboxOff;
            a.seq = c->p2pSeq();
            bool used[2][kMaxDevRanks] = {{false}};
            std::vector<HcclSendRecvItem> later;
            for (const HcclSendRecvItem& it : rest) {
                const int dir = it.sendRecvType == HCCL_SEND ? 0 : 1;
                if (used[dir][it.remoteRank] || a.nItems == kMaxP2pItems) { later.push_back(it); continue; }
                used[dir][it.remoteRank] = true;
                P2pItem& d = a.items[a.nItems++];
                d.buf = (char*)it.buf;
                d.bytes = it.count * DataTypeSize(it.dataType);
                d.peer = (int)it.remoteRank;
                d.isSend = dir == 0;
            }
            CHK_RET(LaunchP2p(tgt, a, std::max(1, a.nItems)));
            rest.swap(later);
            if (p.items.empty()) break;
        }
        return HCCL_SUCCESS;
    }

    HcclResult Run() const
    {
        switch (p.op) {
            case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE: return AllReduceLike();
            case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_REDUCE_SCATTER_V: return dalg == DALG_RS_LL ? LLExchange() : ReduceScatterLike();
            case HCCL_CMD_ALLGATHER: case HCCL_CMD_ALLGATHER_V: return AllGatherLike();
            case HCCL_CMD_BROADCAST: return dalg == DALG_BCAST_LL ? LLExchange() : Broadcast();
            case HCCL_CMD_SCATTER: return Scatter();
            case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: return dalg == DALG_A2A_LL ? LLExchange() : AlltoAllLike();
            case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: case HCCL_CMD_BATCH_SEND_RECV: return PointToPoint();
            case HCCL_CMD_BARRIER: {
                CollArgs a;
                memset(&a, 0, sizeof(a));
                return LaunchCollective(tgt, DALG_BARRIER, HCCL_DATA_TYPE_INT8, a, 1);
            }
            default: return HCCL_E_NOT_SUPPORT;
        }
    }
};

OpDesc Describe(CommImpl* c, const OpParam& p)
{
    OpDesc d;
    d.op = p.op;
    d.dtype = p.dtype;
    d.redOp = p.redOp;
    d.root = p.root;
    d.nRanks = (uint32_t)c->nRanks;
    d.det = c->cfg.deterministic;
    d.engine = c->cfg.engine;
    d.isMc2 = p.isMc2;
    d.castScale = p.castScale;
    d.stageInBytes = c->layout().inBytes;
    const uint64_t es = DataTypeSize(p.dtype);
    const uint64_t P = (uint64_t)c->nRanks;
    const char* peers[kMaxDevRanks];
    uint64_t inBytes = 0, outBytes = 0;
    switch (p.op) {
        case HCCL_CMD_ALLREDUCE: case HCCL_CMD_REDUCE: case HCCL_CMD_BROADCAST: d.bytes = p.count * es; inBytes = outBytes = d.bytes; break;
        case HCCL_CMD_ALLGATHER: d.bytes = p.count * es * P; inBytes = p.count * es; outBytes = d.bytes; break;
        case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_SCATTER: d.bytes = p.count * es * P; inBytes = d.bytes; outBytes = p.count * es; break;
        case HCCL_CMD_ALLGATHER_V: for (uint64_t v : p.recvCounts) d.bytes += v * es; inBytes = p.count * es; outBytes = d.bytes; break;
        case HCCL_CMD_REDUCE_SCATTER_V: for (uint64_t v : p.sendCounts) d.bytes += v * es; inBytes = d.bytes; outBytes = p.count * es; break;
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC:
            for (uint64_t v : p.sendCounts) d.bytes += v * es;
            inBytes = outBytes = d.bytes;
            break;
        case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: d.bytes = p.count * es; break;
        case HCCL_CMD_BATCH_SEND_RECV: for (auto& it : p.items) d.bytes += it.count * DataTypeSize(it.dataType); break;
        default: break;
    }
    const char* mcIn = nullptr;
    const char* mcOut = nullptr;
    d.inRegistered = p.send && inBytes && c->Lookup(p.send, inBytes, peers, &mcIn);
    d.outRegistered = p.recv && outBytes && c->Lookup(p.recv, outBytes, peers, &mcOut);
    d.inMulticast = d.inRegistered && mcIn != nullptr;       // buffers registered with HcclCommRegister have no multicast alias
    d.outMulticast = d.outRegistered && mcOut != nullptr;
    d.aligned16 = Aligned16(p.send) && Aligned16(p.recv);
    // in place: the output overlaps the input (AllGather / ReduceScatter on a slice of the other buffer included)
    const char* sb = (const char*)p.send;
    const char* rb = (const char*)p.recv;
    d.inPlace = sb != nullptr && rb != nullptr && sb < rb + outBytes && rb < sb + inBytes;
    return d;
}

// What identifies a call on every rank alike: everything selection looks at except the facts about this rank's own
// buffers.  AlltoAllV counts are private to a rank, so its size is left out.
uint64_t SharedSignature(const OpParam& p, const OpDesc& d, uint64_t generation)
{
    const bool privateSize = p.op == HCCL_CMD_ALLTOALLV;
    const uint64_t fields[6] = {(uint64_t)p.op, (uint64_t)p.dtype, (uint64_t)p.redOp, (uint64_t)p.root, privateSize ? 0 : d.bytes, generation};
    return Fnv1a(fields, sizeof(fields));
}

bool IsCollective(HcclCMDType op) { return op != HCCL_CMD_SEND && op != HCCL_CMD_RECEIVE && op != HCCL_CMD_BATCH_SEND_RECV; }

// Ranks may be called with buffers that differ in registration, alignment or aliasing, and both the choice of an
// algorithm and its launch shape depend on those facts; ranks that chose differently would wait for flags that never
// come.  So the first time a rank meets a call signature it exchanges its flag word with all ranks (reference: ranks
// exchange their execution configuration and take the lowest common one, op_common.cc:265-276, comm_negotiation.h:
// 41-50) and everything a peer can observe is derived from the combined word, which the plan keeps.  A rank that
// meets the signature with the same local facts again reuses the plan without talking to anybody.
struct ShapeRecord { uint64_t signature; uint32_t flags; uint32_t pad; };
HcclResult AgreeOnCallShape(CommImpl* c, const OpParam& p, uint64_t signature, uint32_t localFlags, uint32_t* agreed)
{
    *agreed = localFlags;
    if (!c->bs || !IsCollective(p.op) || !GetEnvConfig().callShapeAgree) return HCCL_SUCCESS;
    ShapeRecord mine = {signature, localFlags, 0};
    std::vector<ShapeRecord> all((size_t)c->nRanks);
    // A signature met again with other local facts: the peers take part in this exchange only if their facts changed
    // too (ranks that still have the plan reuse it silently).  Say so before waiting, and again if the wait fails.
    const auto seen = c->shapeSeen.find(signature);
    const bool again = seen != c->shapeSeen.end() && seen->second != localFlags;
    if (again)
        HCCL_WARNING("comm %s rank %d: %s met again with other buffer facts (flags %#x, were %#x); the exchange completes only if every rank's "
                     "registration / alignment / aliasing changed with this call", c->name.c_str(), c->rank, CmdName(p.op), localFlags, seen->second);
    const HcclResult xr = c->bs->AllGather(&mine, all.data(), sizeof(mine));
    if (xr != HCCL_SUCCESS) {
        if (again)
            HCCL_ERROR("comm %s rank %d: the buffer facts of %s changed on this rank only (flags %#x, were %#x): its peers reused their plan and did "
                       "not join the exchange.  Change registration, alignment and in-place use on all ranks together, or set "
                       "HCCL_CALL_SHAPE_AGREE=0 when every rank is known to pass equivalent buffers", c->name.c_str(), c->rank, CmdName(p.op), localFlags,
                       seen->second);
        return xr;
    }
    if (c->shapeSeen.size() >= 16384) c->shapeSeen.clear();      // only feeds the diagnosis above
    c->shapeSeen[signature] = localFlags;
    for (int r = 0; r < c->nRanks; ++r) {
        if (all[(size_t)r].signature != signature) {
            HCCL_ERROR("comm %s: rank %d and rank %d are not in the same operation (%s here): operator, data type, reduce op, root or count differ",
                       c->name.c_str(), c->rank, r, CmdName(p.op));
            return HCCL_E_PARA;
        }
        *agreed = OpDesc::CombineFlags(*agreed, all[(size_t)r].flags);
    }
    if (*agreed != localFlags)
        HCCL_RUN_INFO("comm %s rank %d: %s runs on the buffer facts all ranks share (flags %#x, local %#x)", c->name.c_str(), c->rank, CmdName(p.op),
                      *agreed, localFlags);
    return HCCL_SUCCESS;
}

}  // namespace

// Selection (or plan reuse) and execution of a described call.  `presetAgreed` carries the combined flag word when
// the caller already knows it (emulated ranks, whose calls are collected first).
HcclResult ExecDescribed(CommImpl* c, OpParam& p, OpDesc d, const uint32_t* presetAgreed)
{
    const auto t0 = std::chrono::steady_clock::now();
    const uint32_t localFlags = d.Flags();
    // a plan is the outcome of selection: it dies with the communicator's generation and with a reload of the environment
    PlanKey key = {(uint32_t)p.op, (uint32_t)p.dtype, (uint32_t)p.redOp, p.root, d.bytes, localFlags, (uint32_t)c->generation ^ (EnvConfigVersion() << 16)};
    Plan plan;
    const AlgEntry* alg = nullptr;
    // a plan made for other combined flags (emulated ranks: the combination is known before every call and depends on
    // what the OTHER ranks passed, which the key does not see) is replaced
    const bool cacheable = c->cfg.planCacheEnable;
    if (cacheable && c->plans->Find(key, &plan) && (presetAgreed == nullptr || plan.agreedFlags == *presetAgreed)) {
        alg = &AlgRegistry::Instance().All()[(size_t)plan.algIndex];
        d.ApplyFlags(plan.agreedFlags);
    } else {
        uint32_t agreed = localFlags;
        if (presetAgreed != nullptr) agreed = *presetAgreed;
        else CHK_RET(AgreeOnCallShape(c, p, SharedSignature(p, d, c->generation), localFlags, &agreed));
        d.ApplyFlags(agreed);
        Selection sel;
        CHK_RET(SelectAlgorithm(*c->selector, *c->topo, GetEnvConfig(), d, c->name, (HcclComm)c, c->cfg.bufferBytes, &sel));
        alg = sel.alg;
        plan.algIndex = sel.algIndex;
        plan.devAlg = alg->devAlg;
        plan.agreedFlags = agreed;
        if (cacheable) c->plans->Insert(key, plan);
    }
    p.algName = alg->name;
    c->ctx.Put("last_alg", std::vector<uint8_t>(alg->name.begin(), alg->name.end()));
    ProfilingScope prof(c, p, alg->name.c_str(), d.bytes);
    HcclResult r = Exec(c, p, d, alg).Run();
    if (r != HCCL_SUCCESS) HCCL_ERROR("comm %s rank %d: %s with algorithm %s failed: %s", c->name.c_str(), c->rank, CmdName(p.op), alg->name.c_str(), ResultString(r));
    prof.SetHostUs(std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count());
    return r;
}

OpDesc DescribeCall(CommImpl* c, const OpParam& p) { return Describe(c, p); }

struct EmuGroup::PendingOp { OpParam p; };

HcclResult EmuSubmitCollective(CommImpl* c, const OpParam& p)
{
    EmuGroup* g = c->emuGroup();
    std::lock_guard<std::mutex> lk(g->opMu);
    const int n = g->nRanks();
    std::shared_ptr<EmuGroup::PendingOp> mine(new EmuGroup::PendingOp{p});
    g->pendingOps[(size_t)c->rank].push_back(mine);
    HcclResult result = HCCL_SUCCESS;
    for (;;) {
        for (int r = 0; r < n; ++r)
            if (g->pendingOps[(size_t)r].empty()) return result;
        std::vector<std::shared_ptr<EmuGroup::PendingOp>> ops;
        for (int r = 0; r < n; ++r) { ops.push_back(g->pendingOps[(size_t)r].front()); g->pendingOps[(size_t)r].pop_front(); }
        // the same operator everywhere (the multi-process path compares this over the bootstrap on the first call)
        std::vector<OpDesc> descs;
        uint32_t agreed = 0;
        const OpParam& first = ops[0]->p;
        for (int r = 0; r < n; ++r) {
            const OpParam& q = ops[(size_t)r]->p;
            const bool countMustMatch = q.op != HCCL_CMD_ALLTOALLV && q.op != HCCL_CMD_ALLGATHER_V && q.op != HCCL_CMD_REDUCE_SCATTER_V;
            if (q.op != first.op || q.dtype != first.dtype || q.redOp != first.redOp || q.root != first.root || (countMustMatch && q.count != first.count)) {
                HCCL_ERROR("emulated ranks 0 and %d are not in the same operation (%s vs %s, count %llu vs %llu)", r, CmdName(first.op), CmdName(q.op),
                           (unsigned long long)first.count, (unsigned long long)q.count);
                return HCCL_E_PARA;
            }
            descs.push_back(Describe(g->members[(size_t)r], q));
            agreed = r == 0 ? descs.back().Flags() : OpDesc::CombineFlags(agreed, descs.back().Flags());
        }
        for (int r = 0; r < n; ++r) {
            HcclResult e = ExecDescribed(g->members[(size_t)r], ops[(size_t)r]->p, descs[(size_t)r], &agreed);
            if (e != HCCL_SUCCESS) result = e;
        }
    }
}

HcclResult ExecOp(CommImpl* c, OpParam& p)
{
    CHK_PTR_NULL(c);
    CHK_RET(c->CheckReady());
    // ranks emulated on one GPU are called one after the other: their collectives are queued and run together once
    // the last rank has called, when every rank's buffer facts are known (the group's own lock serialises them)
    if (c->emulated() && c->nRanks > 1 && !c->hostComm && IsCollective(p.op)) {
        HcclResult emuErr;
        c->PollAsyncError(&emuErr);
        if (emuErr != HCCL_SUCCESS) return emuErr;
        ++c->opCount;
        return EmuSubmitCollective(c, p);
    }
    std::lock_guard<std::mutex> lk(c->opMu);
    HcclResult asyncErr;
    c->PollAsyncError(&asyncErr);
    if (asyncErr != HCCL_SUCCESS) return asyncErr;
    ++c->opCount;
    if (EntryLogEnabled() || GetEnvConfig().diagnose) {
        std::ostringstream os;
        os << "Entry-Hccl" << CmdName(p.op) << ": tag[" << p.tag << "] sendBuf[" << p.send << "] recvBuf[" << p.recv << "] count[" << p.count
           << "] dataType[" << DataTypeName(p.dtype) << "] op[" << ReduceOpName(p.redOp) << "] root[" << p.root << "] rank[" << c->rank << "/"
           << c->nRanks << "] stream[" << (void*)p.stream << "] comm[" << c->name << "] seq[" << c->opCount << "]";
        HCCL_RUN_INFO("%s", os.str().c_str());
        if (GetEnvConfig().diagnose) DiagnoseRecord(os.str());
    }
    {
        // an algorithm plugin may claim the call before any built-in selection (reference op_common.cc:205-207, :1275-1281)
        HcclResult pr;
        std::string pname;
        if (AlgoPluginTryExecute(c, p, &pr, &pname)) { p.algName = pname; return pr; }
    }
    if (c->hostComm) return HostExecOp(c, p);       // host engine communicators run the algorithm templates on host threads
    if (c->nRanks == 1) return SingleRank(c, p);
    CHK_RET(FirstCallCheck(c, p));
    return ExecDescribed(c, p, Describe(c, p), nullptr);
}

}  // namespace hccl
