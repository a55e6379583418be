// C entry points of the MoE dispatch / combine operators.
#include <cstring>
#include <mutex>
#include "../core/comm.h"
#include "../core/log.h"
#include "../kernels/moe_launch.h"
#include "hccl/hccl_moe.h"

using namespace hccl;

namespace hccl {
// Per-communicator scratch of the MoE kernels: expert counters, pair positions and the symmetric count-exchange table.
struct MoeState {
    uint32_t* counts = nullptr;     // [kMoeMaxExperts]
    uint32_t* pos = nullptr;        // [posCap]
    size_t posCap = 0;
    void* table = nullptr;          // HcclMemAlloc'ed, kMoeTableBytes
    CommImpl* owner = nullptr;
    ~MoeState()
    {
        if (counts) cudaFree(counts);
        if (pos) cudaFree(pos);
    }
};
}  // namespace hccl

namespace {

HcclResult CheckCfg(const CommImpl* c, const HcclMoeConfig* cfg)
{
    if (!cfg) return HCCL_E_PTR;
    if (cfg->hidden == 0 || cfg->hidden % 128 != 0 || cfg->hidden > 8192) { HCCL_ERROR("MoE: hidden must be a multiple of 128 up to 8192 (got %u)", cfg->hidden); return HCCL_E_PARA; }
    if (cfg->topk == 0 || cfg->topk > (uint32_t)kMoeMaxTopk) { HCCL_ERROR("MoE: topk must be 1..%d (got %u)", kMoeMaxTopk, cfg->topk); return HCCL_E_PARA; }
    if (cfg->nExperts == 0 || cfg->nExperts > (uint32_t)kMoeMaxExperts || cfg->nExperts % (uint32_t)c->nRanks != 0) {
        HCCL_ERROR("MoE: the number of experts must be a multiple of the %d ranks, at most %d (got %u)", c->nRanks, kMoeMaxExperts, cfg->nExperts);
        return HCCL_E_PARA;
    }
    if (cfg->capacity == 0) return HCCL_E_PARA;
    return HCCL_SUCCESS;
}

HcclResult EnsureState(CommImpl* c, size_t nPairs)
{
    if (!c->moe) {
        std::shared_ptr<MoeState> st(new MoeState());
        CHK_CUDA(cudaMalloc(&st->counts, sizeof(uint32_t) * kMoeMaxExperts));
        CHK_RET(c->MemAlloc(kMoeTableBytes, &st->table));       // collective: every rank reaches this on its first dispatch
        CHK_CUDA(cudaMemset(st->table, 0, kMoeTableBytes));
        c->moe = st;
    }
    MoeState* st = c->moe.get();
    if (nPairs > st->posCap) {
        if (st->pos) { CHK_CUDA(cudaDeviceSynchronize()); cudaFree(st->pos); st->pos = nullptr; }
        CHK_CUDA(cudaMalloc(&st->pos, sizeof(uint32_t) * nPairs));
        st->posCap = nPairs;
    }
    return HCCL_SUCCESS;
}

int MoeBlocks(const CommImpl* c, uint32_t nTokens)
{
    // combine is a pull over NVLink, bound by the bytes in flight: as many blocks as the flag rows allow
    int nb = (int)std::min<uint32_t>(std::max<uint32_t>(nTokens / 8, 1), 128);
    return std::min(nb, c->MaxBlocks());
}

}  // namespace

extern "C" {

HcclResult HcclMoeDispatch(HcclComm comm, const void* x, const int32_t* topkIdx, const HcclMoeConfig* cfg, void* recvX, void* recvScale, void* recvSrc,
                           uint32_t* recvOffsets, uint64_t* slotMap, hcclStream_t stream)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(x); CHK_PTR_NULL(topkIdx); CHK_PTR_NULL(recvX); CHK_PTR_NULL(recvScale); CHK_PTR_NULL(recvSrc);
    CHK_PTR_NULL(recvOffsets); CHK_PTR_NULL(slotMap);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (c->hostComm) return HCCL_E_NOT_SUPPORT;
    CHK_RET(c->CheckReady());
    CHK_RET(CheckCfg(c, cfg));
    std::lock_guard<std::mutex> lk(c->opMu);
    const size_t nPairs = (size_t)cfg->nTokens * cfg->topk;
    CHK_RET(EnsureState(c, std::max<size_t>(nPairs, 1)));
    MoeState* st = c->moe.get();
    MoeDispatchArgs a;
    memset(&a, 0, sizeof(a));
    const char *px[kMaxDevRanks], *ps[kMaxDevRanks], *pr[kMaxDevRanks], *pt[kMaxDevRanks];
    if (!c->Lookup(recvX, (uint64_t)cfg->capacity * cfg->hidden, px, nullptr) || !c->Lookup(recvScale, (uint64_t)cfg->capacity * (cfg->hidden / 128) * 4, ps, nullptr) ||
        !c->Lookup(recvSrc, (uint64_t)cfg->capacity * 8, pr, nullptr) || !c->Lookup(st->table, kMoeTableBytes, pt, nullptr)) {
        HCCL_ERROR("MoE dispatch: the receive buffers must be symmetric memory (HcclMemAlloc) of at least `capacity` rows");
        return HCCL_E_PARA;
    }
    for (int q = 0; q < c->nRanks; ++q) {
        a.recvX[q] = (uint8_t*)px[q]; a.recvScale[q] = (float*)ps[q]; a.recvSrc[q] = (uint64_t*)pr[q]; a.table[q] = (uint32_t*)pt[q];
    }
    a.x = (const __nv_bfloat16*)x; a.topkIdx = topkIdx; a.counts = st->counts; a.pos = st->pos; a.slotMap = slotMap; a.recvOffsets = recvOffsets;
    a.nTokens = (int)cfg->nTokens; a.hidden = (int)cfg->hidden; a.topk = (int)cfg->topk; a.nExperts = (int)cfg->nExperts; a.capacity = cfg->capacity;
    CHK_RET(LaunchMoeCount(topkIdx, (int)nPairs, (int)cfg->nExperts, st->counts, st->pos, (cudaStream_t)stream));
    // every rank launches the same grid: sized by a value all ranks share (the configured token count must match)
    return LaunchMoeDispatch(c->Target((cudaStream_t)stream), a, MoeBlocks(c, cfg->nTokens));
}

HcclResult HcclMoeCombine(HcclComm comm, const void* y, const float* topkWeight, const uint64_t* slotMap, const HcclMoeConfig* cfg, void* out,
                          hcclStream_t stream)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(y); CHK_PTR_NULL(topkWeight); CHK_PTR_NULL(slotMap); CHK_PTR_NULL(out);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (c->hostComm) return HCCL_E_NOT_SUPPORT;
    CHK_RET(c->CheckReady());
    CHK_RET(CheckCfg(c, cfg));
    std::lock_guard<std::mutex> lk(c->opMu);
    MoeCombineArgs a;
    memset(&a, 0, sizeof(a));
    const char* py[kMaxDevRanks];
    if (!c->Lookup(y, (uint64_t)cfg->capacity * cfg->hidden * 2, py, nullptr)) {
        HCCL_ERROR("MoE combine: the expert output buffer must be symmetric memory (HcclMemAlloc) of `capacity` rows");
        return HCCL_E_PARA;
    }
    for (int q = 0; q < c->nRanks; ++q) a.y[q] = (const __nv_bfloat16*)py[q];
    a.topkWeight = topkWeight; a.slotMap = slotMap; a.out = (__nv_bfloat16*)out;
    a.nTokens = (int)cfg->nTokens; a.hidden = (int)cfg->hidden; a.topk = (int)cfg->topk; a.capacity = cfg->capacity;
    return LaunchMoeCombine(c->Target((cudaStream_t)stream), a, MoeBlocks(c, cfg->nTokens));
}

}  // extern "C"
