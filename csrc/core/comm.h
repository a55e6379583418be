// The communicator object: rank identity, effective configuration, bootstrap
// connection, the symmetric slab (flags + LL region + staging), registered user
// segments, device-side communicator view, status block and caches.
//
// HCCL keeps this in HCOMM (communicator, EngineCtx key/value store, thread and
// channel resources); the operator layer reaches it through HcclEngineCtxCreate/
// Get (op_common.cc:1846-1876) and HcclGetHcclBuffer.  Here it is one C++ class.
#pragma once
#include <atomic>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include <cuda_runtime.h>
#include "bootstrap.h"
#include "config.h"
#include "symmem.h"
#include "hccl/hccl_types.h"
#include "../kernels/launch.h"

namespace hccl {

struct DevComm;
struct DevStatus;
class EmuGroup;
struct TopoInfo;
class SelectorState;
class PlanCache;
class HostRank;
struct Mc2State;
struct MoeState;

// Named blobs owned by the communicator (topology cache, cost model, tuner
// context, fallback records) - the EngineCtx store of the reference.
class CtxStore {
public:
    bool Get(const std::string& tag, std::vector<uint8_t>* out) const;
    void Put(const std::string& tag, std::vector<uint8_t> blob);
    void Erase(const std::string& tag);
    void Clear();
    size_t size() const;
private:
    mutable std::mutex mu_;
    std::map<std::string, std::vector<uint8_t>> blobs_;
};

struct StageLayout {
    uint64_t dataBytes;     // whole staging data region
    uint64_t inOff, inBytes;     // stage-in region
    uint64_t xchOff, xchBytes;   // exchange region (phase-2 sources, metadata tables)
    uint64_t mailboxOff, mailboxHalf;  // p2p mailboxes: [from][2][half]
};

// How a staging slab of dataBytes is divided among stage-in region, exchange region and p2p mailboxes for nRanks ranks.
StageLayout MakeStageLayout(uint64_t dataBytes, int nRanks);

class CommImpl {
public:
    CommImpl();
    ~CommImpl();

    // multi-process / multi-thread initialisation: one rank per GPU
    HcclResult Init(const HcclRootInfo& root, int nRanks, int rank, const HcclCommConfig* cfg);
    // emulation: called by EmuGroup for each rank
    HcclResult InitEmulated(EmuGroup* group, int nRanks, int rank, const SymSegment& slab, const HcclCommConfig* cfg);
    HcclResult Destroy();

    HcclResult CheckReady() const;                 // READY else HCCL_E_SUSPENDING / error
    HcclResult PollAsyncError(HcclResult* out);    // reads the status block
    std::string DescribeAsyncError() const;
    HcclResult Suspend();
    HcclResult Resume();                           // collective: clears flags / epochs, bumps generation

    // symmetric user memory
    HcclResult MemAlloc(uint64_t size, void** ptr);
    HcclResult MemFree(void* ptr);
    HcclResult RegisterBuffer(void* ptr, uint64_t size);     // collective: a buffer the caller allocated itself
    HcclResult DeregisterBuffer(void* ptr);
    // Finds the registered segment covering [p, p+bytes); fills peer pointers. false if not registered.
    bool Lookup(const void* p, uint64_t bytes, const char* peerPtr[HCCL_MAX_DEVICE_RANKS], const char** mcPtr) const;

    LaunchTarget Target(cudaStream_t stream) const;
    const DevComm& dev() const { return *dev_; }
    DevStatus* status() const { return hStatus_; }
    uint64_t* p2pSeq() const { return dP2pSeq_; }
    char* StageBase(int rank) const;    // rank r's staging data region as mapped here
    char* StageMcBase() const;
    const StageLayout& layout() const { return layout_; }
    bool nvls() const { return slab_.mc != nullptr; }
    bool emulated() const { return emu_ != nullptr; }
    EmuGroup* emuGroup() const { return emu_; }
    int MaxBlocks() const;

    int rank = 0, nRanks = 1, device = 0;
    std::string name;
    EffectiveConfig cfg;
    std::atomic<int> status_{HCCL_COMM_STATUS_READY};
    uint64_t generation = 0;       // bumped by Resume; cached plans are keyed by it
    uint64_t opCount = 0;
    CtxStore ctx;
    std::unique_ptr<Bootstrap> bs;
    std::mutex opMu;               // serialises op submission on this communicator
    std::unique_ptr<SelectorState> selector;
    std::unique_ptr<PlanCache> plans;
    std::unique_ptr<TopoInfo> topo;
    bool firstOpChecked[HCCL_CMD_MAX] = {false};
    std::map<uint64_t, uint32_t> shapeSeen;   // call signature -> the local buffer facts it was last agreed with
    std::shared_ptr<MoeState> moe;  // scratch of the MoE dispatch / combine kernels, created on first use
    std::shared_ptr<Mc2State> mc2;  // resources of the fused matmul kernels, created on first use
    HostRank* hostComm = nullptr;  // non-null: a host-engine communicator (ranks are host threads)

private:
    HcclResult SetupDeviceState();
    SymSegment slab_;
    bool ownsSlab_ = true;
    std::vector<SymSegment> userSegs_;
    DevComm* dev_ = nullptr;        // host copy (heap)
    uint64_t* dEpochs_ = nullptr;
    uint32_t* dAbort_ = nullptr;
    uint64_t* dP2pSeq_ = nullptr;
    DevStatus* hStatus_ = nullptr;  // pinned, mapped
    DevStatus* dStatus_ = nullptr;  // device alias of hStatus_
    EmuGroup* emu_ = nullptr;
    StageLayout layout_{};
    // watchdog (stuck detection): compares head/tail of the status block
    std::thread watchdog_;
    std::atomic<bool> watchdogStop_{false};
    void WatchdogLoop();
public:
    std::atomic<uint64_t> stuckReports{0};
};

// Process-wide registry of communicators by name, for callers that know a group only by its name (graph mode).
void GroupRegister(CommImpl* c);
void GroupUnregister(CommImpl* c);
// All live communicators named `name` in this process.
std::vector<CommImpl*> GroupFind(const std::string& name);

// Ranks that share one GPU inside one process.  Collects each rank's launch and
// issues ONE cooperative kernel when the last rank has posted.
class EmuGroup : public EmuLauncher {
public:
    static HcclResult Create(int nRanks, const HcclCommConfig* cfg, std::vector<CommImpl*>* comms);
    ~EmuGroup() override;
    HcclResult Post(int rank, const void* args, size_t argBytes, int nBlocks, int threads, const void* emuKernel,
                    cudaStream_t stream) override;
    HcclResult MemAlloc(int rank, uint64_t size, SymSegment* seg);   // R matching calls -> one group allocation
    void Release(CommImpl* c);
    int nRanks() const { return nRanks_; }
    // Collectives queued per rank until every rank has called (the operator layer owns the entries).
    struct PendingOp;
    std::mutex opMu;
    std::vector<std::deque<std::shared_ptr<PendingOp>>> pendingOps;
    std::vector<CommImpl*> members;
private:
    EmuGroup() = default;
    int nRanks_ = 0;
    int alive_ = 0;
    std::mutex mu_;
    DevComm* dComms_ = nullptr;            // device array [nRanks]
    // ring of argument slots (pinned host + device), each holds nRanks * kArgSlotBytes
    static constexpr int kRing = 64;
    static constexpr size_t kArgSlotBytes = 4096;
    char* hArgs_ = nullptr;
    char* dArgs_ = nullptr;
    cudaEvent_t ringEvents_[kRing] = {nullptr};
    int ringHead_ = 0;
    // launches posted by individual ranks and not yet issued
    struct PendingPost { const void* kernel; int nBlocks, threads; std::vector<char> args; };
    std::vector<std::deque<PendingPost>> queues_;
    std::vector<DevComm> hostComms_;
    // pending group allocation
    std::vector<std::vector<SymSegment>> allocRounds_;
    std::vector<size_t> allocNext_;
    friend class CommImpl;
    std::vector<SymSegment> slabs_;
    int maxBlocksPerRank_ = 1;
};

}  // namespace hccl
