#include "comm.h"
#include <algorithm>
#include <chrono>
#include <cstring>
#include "../kernels/dev_types.h"
#include "../select/selector.h"
#include "../topo/topo.h"
#include "log.h"
#include "plan_cache.h"
#include "../cpu/host_comm.h"

namespace hccl {

// ---------------------------------------------------------------- CtxStore
bool CtxStore::Get(const std::string& tag, std::vector<uint8_t>* out) const
{
    std::lock_guard<std::mutex> lk(mu_);
    auto it = blobs_.find(tag);
    if (it == blobs_.end()) return false;
    if (out) *out = it->second;
    return true;
}
void CtxStore::Put(const std::string& tag, std::vector<uint8_t> blob)
{
    std::lock_guard<std::mutex> lk(mu_);
    blobs_[tag] = std::move(blob);
}
void CtxStore::Erase(const std::string& tag)
{
    std::lock_guard<std::mutex> lk(mu_);
    blobs_.erase(tag);
}
void CtxStore::Clear()
{
    std::lock_guard<std::mutex> lk(mu_);
    blobs_.clear();
}
size_t CtxStore::size() const
{
    std::lock_guard<std::mutex> lk(mu_);
    return blobs_.size();
}

// ---------------------------------------------------------------- CommImpl
CommImpl::CommImpl() : dev_(new DevComm()) { memset(dev_, 0, sizeof(DevComm)); }

CommImpl::~CommImpl()
{
    Destroy();
    delete dev_;
}

StageLayout MakeStageLayout(uint64_t dataBytes, int nRanks)
{
    StageLayout l{};
    l.dataBytes = dataBytes;
    // p2p mailboxes take 1/8 of the slab at most (two halves per sender), at least 64 KiB per half
    uint64_t half = dataBytes / 8 / (2ull * (uint64_t)nRanks);
    half = half > (4ull << 20) ? (4ull << 20) : half;
    half &= ~(uint64_t)4095;
    if (half < 65536) half = 65536;
    const uint64_t mailbox = half * 2 * (uint64_t)nRanks;
    l.mailboxHalf = half;
    l.mailboxOff = (dataBytes - mailbox) & ~(uint64_t)4095;
    const uint64_t rest = l.mailboxOff;
    l.inOff = 0;
    l.inBytes = (rest / 2) & ~(uint64_t)4095;
    l.xchOff = l.inBytes;
    l.xchBytes = (rest - l.inBytes) & ~(uint64_t)4095;
    return l;
}

HcclResult CommImpl::SetupDeviceState()
{
    CHK_CUDA(cudaMalloc(&dEpochs_, kEpochWords * sizeof(uint64_t)));
    CHK_CUDA(cudaMemset(dEpochs_, 0, kEpochWords * sizeof(uint64_t)));
    CHK_CUDA(cudaMalloc(&dAbort_, 256));
    CHK_CUDA(cudaMemset(dAbort_, 0, 256));
    CHK_CUDA(cudaMalloc(&dP2pSeq_, 2 * kMaxDevRanks * sizeof(uint64_t)));
    CHK_CUDA(cudaMemset(dP2pSeq_, 0, 2 * kMaxDevRanks * sizeof(uint64_t)));
    CHK_CUDA(cudaHostAlloc((void**)&hStatus_, sizeof(DevStatus), cudaHostAllocMapped | cudaHostAllocPortable));
    memset((void*)hStatus_, 0, sizeof(DevStatus));
    CHK_CUDA(cudaHostGetDevicePointer((void**)&dStatus_, (void*)hStatus_, 0));
    dev_->rank = rank;
    dev_->nRanks = nRanks;
    for (int q = 0; q < nRanks; ++q) dev_->slab[q] = (char*)slab_.peer[q];
    dev_->slabMc = (char*)slab_.mc;
    dev_->epochs = dEpochs_;
    dev_->abortWord = dAbort_;
    dev_->status = dStatus_;
    dev_->timeoutNs = cfg.execTimeoutNs;
    dev_->stageBytes = slab_.size - kSlabDataOff;
    layout_ = MakeStageLayout(dev_->stageBytes, nRanks);
    CHK_CUDA(cudaDeviceSynchronize());
    selector.reset(new SelectorState());
    plans.reset(new PlanCache());
    return HCCL_SUCCESS;
}

HcclResult CommImpl::Init(const HcclRootInfo& root, int nR, int r, const HcclCommConfig* config)
{
    const EnvConfig& env = GetEnvConfig();
    CHK_RET(MergeConfig(env, config, &cfg));
    rank = r;
    nRanks = nR;
    if (nRanks > kMaxDevRanks) {
        HCCL_ERROR("this build drives one NVSwitch domain of at most %d GPUs (got %d ranks)", kMaxDevRanks, nRanks);
        return HCCL_E_NOT_SUPPORT;
    }
    CHK_CUDA(cudaGetDevice(&device));
    bs.reset(new Bootstrap());
    CHK_RET(bs->Connect(root, rank, nRanks, env.connectTimeoutS));
    char nm[HCCL_COMM_CONFIG_NAME_MAX];
    snprintf(nm, sizeof(nm), "hccl_comm_%016llx", (unsigned long long)bs->uniqueId());
    name = cfg.commName.empty() ? nm : cfg.commName;
    GroupRegister(this);
    const size_t slabBytes = kSlabDataOff + cfg.bufferBytes;
    const bool wantMc = cfg.nvlsEnable != 0 && nRanks > 1;
    CHK_RET(SymAlloc(*bs, device, slabBytes, wantMc, env.forceIpc, &slab_));
    if (cfg.nvlsEnable == 1 && nRanks > 1 && slab_.mc == nullptr)
        HCCL_WARNING("NVLS was requested but the box does not expose multicast: using P2P kernels");
    CHK_RET(SetupDeviceState());
    topo.reset(new TopoInfo());
    CHK_RET(DiscoverTopo(this, topo.get()));
    HCCL_CONFIG_INFO(LOG_MOD_RESOURCE,
                     "comm %s rank %d/%d device %d: slab %zu MiB via %s, NVLS %s, stage-in %llu MiB, exchange %llu MiB, "
                     "mailbox half %llu KiB, wait budget %.1f s",
                     name.c_str(), rank, nRanks, device, slabBytes >> 20,
                     slab_.transport == SymTransport::VMM ? "VMM" : "IPC", slab_.mc ? "on" : "off",
                     (unsigned long long)(layout_.inBytes >> 20), (unsigned long long)(layout_.xchBytes >> 20),
                     (unsigned long long)(layout_.mailboxHalf >> 10), cfg.execTimeoutNs * 1e-9);
    if (env.dfs.stuckDetection) watchdog_ = std::thread([this] { WatchdogLoop(); });
    return bs->Barrier();
}

HcclResult CommImpl::InitEmulated(EmuGroup* group, int nR, int r, const SymSegment& slab, const HcclCommConfig* config)
{
    const EnvConfig& env = GetEnvConfig();
    CHK_RET(MergeConfig(env, config, &cfg));
    rank = r;
    nRanks = nR;
    CHK_CUDA(cudaGetDevice(&device));
    emu_ = group;
    slab_ = slab;
    ownsSlab_ = true;
    char nm[HCCL_COMM_CONFIG_NAME_MAX];
    snprintf(nm, sizeof(nm), "hccl_emu_%p", (void*)group);
    name = cfg.commName.empty() ? nm : cfg.commName;
    GroupRegister(this);
    CHK_RET(SetupDeviceState());
    topo.reset(new TopoInfo());
    CHK_RET(DiscoverTopo(this, topo.get()));
    return HCCL_SUCCESS;
}

namespace {
std::mutex g_groupMu;
std::vector<CommImpl*>& Groups()
{
    static std::vector<CommImpl*> v;
    return v;
}
}  // namespace
void GroupRegister(CommImpl* c)
{
    std::lock_guard<std::mutex> lk(g_groupMu);
    auto& v = Groups();
    if (std::find(v.begin(), v.end(), c) == v.end()) v.push_back(c);
}
void GroupUnregister(CommImpl* c)
{
    std::lock_guard<std::mutex> lk(g_groupMu);
    auto& v = Groups();
    v.erase(std::remove(v.begin(), v.end(), c), v.end());
}
std::vector<CommImpl*> GroupFind(const std::string& name)
{
    std::lock_guard<std::mutex> lk(g_groupMu);
    std::vector<CommImpl*> out;
    for (CommImpl* c : Groups())
        if (c->name == name) out.push_back(c);
    return out;
}

HcclResult CommImpl::Destroy()
{
    if (status_.load() == HCCL_COMM_STATUS_DESTROYED) return HCCL_SUCCESS;
    status_.store(HCCL_COMM_STATUS_DESTROYED);
    GroupUnregister(this);
    watchdogStop_.store(true);
    if (watchdog_.joinable()) watchdog_.join();
    if (hStatus_ || dEpochs_) cudaDeviceSynchronize();
    // Leave together: a peer must not unmap memory another rank's kernel may still touch.
    if (bs) bs->Barrier();
    for (auto& s : userSegs_) SymFree(&s);
    userSegs_.clear();
    if (ownsSlab_) SymFree(&slab_);
    if (dEpochs_) cudaFree(dEpochs_);
    if (dAbort_) cudaFree(dAbort_);
    if (dP2pSeq_) cudaFree(dP2pSeq_);
    if (hStatus_) cudaFreeHost((void*)hStatus_);
    dEpochs_ = nullptr; dAbort_ = nullptr; dP2pSeq_ = nullptr; hStatus_ = nullptr;
    if (bs) bs->Close();
    ctx.Clear();
    if (emu_) emu_->Release(this);
    emu_ = nullptr;
    if (hostComm) HostRankRelease(hostComm);
    hostComm = nullptr;
    return HCCL_SUCCESS;
}

HcclResult CommImpl::CheckReady() const
{
    switch (status_.load()) {
        case HCCL_COMM_STATUS_READY: return HCCL_SUCCESS;
        case HCCL_COMM_STATUS_SUSPENDING: return HCCL_E_SUSPENDING;
        case HCCL_COMM_STATUS_ERROR: return HCCL_E_REMOTE;
        default: return HCCL_E_PARA;
    }
}

std::string CommImpl::DescribeAsyncError() const
{
    if (!hStatus_ || hStatus_->error == DEV_OK) return "";
    char buf[320];
    // The analogue of the reference's exception decode that prints which rank / flag a stuck kernel waited on
    // (hccl_aiv_utils.cc:360-465).
    snprintf(buf, sizeof(buf),
             "comm %s rank %u: kernel family %u, block row %u gave up waiting on flag slot %u for rank %u "
             "(expected >= %llu, last seen %llu) after %.2f s; ops started %llu, finished %llu",
             name.c_str(), hStatus_->rank, hStatus_->kernelId, hStatus_->block, hStatus_->slot, hStatus_->peer,
             (unsigned long long)hStatus_->expected, (unsigned long long)hStatus_->seen, cfg.execTimeoutNs * 1e-9,
             (unsigned long long)hStatus_->head, (unsigned long long)hStatus_->tail);
    return buf;
}

HcclResult CommImpl::PollAsyncError(HcclResult* out)
{
    *out = HCCL_SUCCESS;
    if (!hStatus_) return HCCL_SUCCESS;
    const uint32_t e = hStatus_->error;
    if (e == DEV_OK) return HCCL_SUCCESS;
    *out = (e == DEV_ERR_TIMEOUT) ? HCCL_E_TIMEOUT : HCCL_E_INTERNAL;
    int expect = HCCL_COMM_STATUS_READY;
    if (status_.compare_exchange_strong(expect, HCCL_COMM_STATUS_ERROR)) HCCL_ERROR("%s", DescribeAsyncError().c_str());
    return HCCL_SUCCESS;
}

HcclResult CommImpl::Suspend()
{
    int expect = HCCL_COMM_STATUS_READY;
    status_.compare_exchange_strong(expect, HCCL_COMM_STATUS_SUSPENDING);
    return HCCL_SUCCESS;
}

HcclResult CommImpl::Resume()
{
    if (status_.load() == HCCL_COMM_STATUS_DESTROYED) return HCCL_E_PARA;
    // All ranks arrive with no kernel in flight, clear their flags, epochs, sequence numbers and status, and leave
    // together.  Cached plans and selector state are dropped (reference: state callbacks clearing caches on resume,
    // stuck_detect_counter_helper.h:168-205).
    CHK_CUDA(cudaDeviceSynchronize());
    if (bs) CHK_RET(bs->Barrier());
    CHK_CUDA(cudaMemset(slab_.peer[rank], 0, kSlabDataOff));
    CHK_CUDA(cudaMemset(dEpochs_, 0, kEpochWords * sizeof(uint64_t)));
    CHK_CUDA(cudaMemset(dAbort_, 0, 256));
    CHK_CUDA(cudaMemset(dP2pSeq_, 0, 2 * kMaxDevRanks * sizeof(uint64_t)));
    memset((void*)hStatus_, 0, sizeof(DevStatus));
    CHK_CUDA(cudaDeviceSynchronize());
    if (bs) CHK_RET(bs->Barrier());
    ++generation;
    if (plans) plans->Clear();
    shapeSeen.clear();
    ctx.Clear();
    if (selector) selector.reset(new SelectorState());
    status_.store(HCCL_COMM_STATUS_READY);
    return HCCL_SUCCESS;
}

char* CommImpl::StageBase(int r) const { return (char*)slab_.peer[r] + kSlabDataOff; }
char* CommImpl::StageMcBase() const { return slab_.mc ? (char*)slab_.mc + kSlabDataOff : nullptr; }

LaunchTarget CommImpl::Target(cudaStream_t stream) const
{
    LaunchTarget t;
    t.dev = dev_;
    t.stream = stream;
    t.emu = emu_;
    t.emuRank = rank;
    return t;
}

int CommImpl::MaxBlocks() const
{
    int m = cfg.maxBlocks ? (int)cfg.maxBlocks : 128;
    if (m > kMaxBlocks) m = kMaxBlocks;
    if (emu_) {
        int cap = emu_->maxBlocksPerRank_;
        if (m > cap) m = cap;
    }
    return m;
}

HcclResult CommImpl::MemAlloc(uint64_t size, void** ptr)
{
    CHK_PTR_NULL(ptr);
    if (size == 0) return HCCL_E_PARA;
    SymSegment seg;
    if (emu_) {
        CHK_RET(emu_->MemAlloc(rank, size, &seg));
    } else {
        // the size must agree: a mismatch would map windows of different sizes
        std::vector<uint64_t> sizes((size_t)nRanks);
        CHK_RET(bs->AllGather(&size, sizes.data(), sizeof(size)));
        for (uint64_t s : sizes)
            if (s != size) { HCCL_ERROR("HcclMemAlloc: ranks passed different sizes (%llu vs %llu)", (unsigned long long)size, (unsigned long long)s); return HCCL_E_PARA; }
        CHK_RET(SymAlloc(*bs, device, size, slab_.mc != nullptr, GetEnvConfig().forceIpc, &seg));
    }
    *ptr = seg.peer[rank];
    userSegs_.push_back(seg);
    return HCCL_SUCCESS;
}

HcclResult CommImpl::MemFree(void* ptr)
{
    for (size_t i = 0; i < userSegs_.size(); ++i) {
        if (userSegs_[i].peer[rank] == ptr) {
            CHK_CUDA(cudaDeviceSynchronize());
            if (bs) CHK_RET(bs->Barrier());
            SymFree(&userSegs_[i]);
            userSegs_.erase(userSegs_.begin() + (long)i);
            return HCCL_SUCCESS;
        }
    }
    HCCL_ERROR("HcclMemFree: %p was not returned by HcclMemAlloc on this communicator", ptr);
    return HCCL_E_NOT_FOUND;
}

HcclResult CommImpl::RegisterBuffer(void* ptr, uint64_t size)
{
    CHK_PTR_NULL(ptr);
    if (size == 0) return HCCL_E_PARA;
    if (emu_ || hostComm || nRanks == 1 || bs == nullptr) return HCCL_E_NOT_SUPPORT;
    const char* peers[HCCL_MAX_DEVICE_RANKS];
    if (Lookup(ptr, size, peers, nullptr)) return HCCL_SUCCESS;        // already symmetric (HcclMemAlloc) or registered
    SymSegment seg;
    CHK_RET(SymRegisterUser(*bs, ptr, size, &seg));
    userSegs_.push_back(seg);
    return HCCL_SUCCESS;
}

HcclResult CommImpl::DeregisterBuffer(void* ptr)
{
    for (size_t i = 0; i < userSegs_.size(); ++i) {
        if (userSegs_[i].peer[rank] == ptr && userSegs_[i].transport == SymTransport::USER_IPC) {
            CHK_CUDA(cudaDeviceSynchronize());
            if (bs) CHK_RET(bs->Barrier());       // no peer still reads the buffer
            SymFree(&userSegs_[i]);
            userSegs_.erase(userSegs_.begin() + (long)i);
            return HCCL_SUCCESS;
        }
    }
    HCCL_ERROR("HcclCommDeregister: %p was not registered on this communicator", ptr);
    return HCCL_E_NOT_FOUND;
}

bool CommImpl::Lookup(const void* p, uint64_t bytes, const char* peerPtr[HCCL_MAX_DEVICE_RANKS], const char** mcPtr) const
{
    for (const SymSegment& s : userSegs_) {
        if (!s.ContainsLocal(p, bytes)) continue;
        const size_t off = (size_t)((const char*)p - (const char*)s.peer[rank]);
        for (int q = 0; q < nRanks; ++q) {
            const void* base = s.peer[q];
            if (!base) return false;
            peerPtr[q] = (const char*)base + off;
        }
        if (mcPtr) *mcPtr = s.mc ? (const char*)s.mc + off : nullptr;
        return true;
    }
    return false;
}

void CommImpl::WatchdogLoop()
{
    // head != tail with no progress for a whole wait budget = an op is stuck between its start and its end
    // (reference: per-communicator head/tail counters compared by a host watchdog, stuck_detect_counter_helper.h).
    uint64_t lastHead = 0, lastTail = 0;
    auto lastChange = std::chrono::steady_clock::now();
    while (!watchdogStop_.load()) {
        for (int i = 0; i < 10 && !watchdogStop_.load(); ++i) std::this_thread::sleep_for(std::chrono::milliseconds(100));
        if (!hStatus_) continue;
        const uint64_t h = hStatus_->head, t = hStatus_->tail;
        auto now = std::chrono::steady_clock::now();
        if (h != lastHead || t != lastTail) { lastHead = h; lastTail = t; lastChange = now; continue; }
        if (h != t) {
            const double idle = std::chrono::duration<double>(now - lastChange).count();
            if (idle * 1e9 > (double)DeriveTimeouts(cfg.execTimeoutNs).fullNs) {
                stuckReports.fetch_add(1);
                HCCL_ERROR("comm %s rank %d: stuck detection: %llu ops started, %llu finished, no progress for %.0f s",
                           name.c_str(), rank, (unsigned long long)h, (unsigned long long)t, idle);
                lastChange = now;
            }
        }
    }
}

// ---------------------------------------------------------------- EmuGroup
HcclResult EmuGroup::Create(int nRanks, const HcclCommConfig* cfg, std::vector<CommImpl*>* comms)
{
    if (nRanks < 1 || nRanks > kMaxDevRanks) return HCCL_E_PARA;
    std::unique_ptr<EmuGroup> g(new EmuGroup());
    g->nRanks_ = nRanks;
    g->alive_ = nRanks;
    g->queues_.resize((size_t)nRanks);
    g->pendingOps.resize((size_t)nRanks);
    EffectiveConfig eff;
    CHK_RET(MergeConfig(GetEnvConfig(), cfg, &eff));
    // emulated ranks share one GPU: keep the per-rank slab modest unless configured
    uint64_t data = (cfg && cfg->hcclBufferSize) || GetEnvConfig().bufferSizeMiB ? eff.bufferBytes : (64ull << 20);
    CHK_RET(SymAllocLocalGroup(nRanks, kSlabDataOff + data, &g->slabs_));
    g->maxBlocksPerRank_ = EmuMaxBlocksPerRank(nRanks);
    CHK_CUDA(cudaMalloc(&g->dComms_, sizeof(DevComm) * (size_t)nRanks));
    CHK_CUDA(cudaHostAlloc((void**)&g->hArgs_, kRing * kArgSlotBytes * (size_t)nRanks, cudaHostAllocDefault));
    CHK_CUDA(cudaMalloc(&g->dArgs_, kRing * kArgSlotBytes * (size_t)nRanks));
    for (int i = 0; i < kRing; ++i) CHK_CUDA(cudaEventCreateWithFlags(&g->ringEvents_[i], cudaEventDisableTiming));
    comms->clear();
    g->hostComms_.resize((size_t)nRanks);
    for (int r = 0; r < nRanks; ++r) {
        CommImpl* c = new CommImpl();
        HcclResult res = c->InitEmulated(g.get(), nRanks, r, g->slabs_[r], cfg);
        if (res != HCCL_SUCCESS) { delete c; return res; }
        g->hostComms_[r] = c->dev();
        g->members.push_back(c);
        comms->push_back(c);
    }
    CHK_CUDA(cudaMemcpy(g->dComms_, g->hostComms_.data(), sizeof(DevComm) * (size_t)nRanks, cudaMemcpyHostToDevice));
    g.release();
    return HCCL_SUCCESS;
}

EmuGroup::~EmuGroup()
{
    cudaDeviceSynchronize();
    if (dComms_) cudaFree(dComms_);
    if (hArgs_) cudaFreeHost(hArgs_);
    if (dArgs_) cudaFree(dArgs_);
    for (int i = 0; i < kRing; ++i) if (ringEvents_[i]) cudaEventDestroy(ringEvents_[i]);
}

void EmuGroup::Release(CommImpl*)
{
    bool last;
    {
        std::lock_guard<std::mutex> lk(mu_);
        last = (--alive_ == 0);
    }
    if (last) delete this;
}

HcclResult EmuGroup::Post(int rank, const void* args, size_t argBytes, int nBlocks, int threads, const void* kernel,
                          cudaStream_t stream)
{
    std::lock_guard<std::mutex> lk(mu_);
    if (argBytes > kArgSlotBytes || rank < 0 || rank >= nRanks_) return HCCL_E_INTERNAL;
    // One FIFO per rank: a rank may run ahead (an operator that needs several loops posts several launches before
    // the next rank is called); a launch is issued whenever every rank has an entry at the head of its queue.
    PendingPost post;
    post.kernel = kernel; post.nBlocks = nBlocks; post.threads = threads;
    post.args.assign((const char*)args, (const char*)args + argBytes);
    queues_[(size_t)rank].push_back(std::move(post));
    for (;;) {
        for (int r = 0; r < nRanks_; ++r)
            if (queues_[(size_t)r].empty()) return HCCL_SUCCESS;
        const PendingPost& first = queues_[0].front();
        for (int r = 1; r < nRanks_; ++r) {
            const PendingPost& o = queues_[(size_t)r].front();
            if (o.kernel != first.kernel || o.nBlocks != first.nBlocks || o.args.size() != first.args.size()) {
                HCCL_ERROR("emulated ranks posted different operations (rank %d differs from rank 0)", r);
                for (auto& q : queues_) q.clear();
                return HCCL_E_PARA;
            }
        }
        const size_t ab = first.args.size();
        int nb = first.nBlocks;
        if (nb > maxBlocksPerRank_) {
            HCCL_ERROR("emulated launch needs %d blocks per rank, only %d fit one cooperative grid", nb, maxBlocksPerRank_);
            for (auto& q : queues_) q.clear();
            return HCCL_E_INTERNAL;
        }
        // the slot is free once the launch that used it last has consumed its arguments
        if (cudaEventQuery(ringEvents_[ringHead_]) == cudaErrorNotReady) CHK_CUDA(cudaEventSynchronize(ringEvents_[ringHead_]));
        char* slot = hArgs_ + (size_t)ringHead_ * kArgSlotBytes * (size_t)nRanks_;
        char* dslot = dArgs_ + (size_t)ringHead_ * kArgSlotBytes * (size_t)nRanks_;
        for (int r = 0; r < nRanks_; ++r) memcpy(slot + (size_t)r * ab, queues_[(size_t)r].front().args.data(), ab);
        const void* fn = first.kernel;
        const int th = first.threads;
        for (auto& q : queues_) q.pop_front();
        CHK_CUDA(cudaMemcpyAsync(dslot, slot, ab * (size_t)nRanks_, cudaMemcpyHostToDevice, stream));
        const DevComm* dc = dComms_;
        const void* da = dslot;
        void* kargs[3] = {(void*)&dc, (void*)&da, (void*)&nb};
        cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3((unsigned)(nb * nRanks_)), dim3((unsigned)th), kargs, 0, stream);
        if (e != cudaSuccess) { HCCL_ERROR("cooperative launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
        CHK_CUDA(cudaEventRecord(ringEvents_[ringHead_], stream));
        ringHead_ = (ringHead_ + 1) % kRing;
    }
}

HcclResult EmuGroup::MemAlloc(int rank, uint64_t size, SymSegment* seg)
{
    std::lock_guard<std::mutex> lk(mu_);
    // Rank r's k-th allocation pairs with every other rank's k-th allocation, whatever the interleaving of the calls.
    // The first rank to reach round k allocates all copies, so that peer pointers are known at once.
    if (allocNext_.empty()) allocNext_.assign((size_t)nRanks_, 0);
    const size_t k = allocNext_[(size_t)rank]++;
    if (k == allocRounds_.size()) {
        allocRounds_.emplace_back();
        CHK_RET(SymAllocLocalGroup(nRanks_, size, &allocRounds_.back()));
    } else if (allocRounds_[k][0].size != size) {
        HCCL_ERROR("HcclMemAlloc: emulated ranks passed different sizes for their allocation number %zu", k);
        return HCCL_E_PARA;
    }
    *seg = allocRounds_[k][(size_t)rank];
    return HCCL_SUCCESS;
}

}  // namespace hccl
