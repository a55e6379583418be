// C entry points for communicator management.
#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <thread>
#include <vector>
#include "../core/algo_plugin.h"
#include "../core/comm.h"
#include "../core/plan_cache.h"
#include "../core/log.h"
#include "../cpu/host_comm.h"
#include "../kernels/dev_types.h"
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "../ops/profiling.h"
#include "../select/selector.h"
#include "hccl/hccl.h"
#include "hccl/hccl_ext.h"
#include "ranktable.h"

using namespace hccl;

extern "C" {

const char* HcclGetVersion(void) { return "hccl_b200 0.1.0"; }
HcclResult HcclReloadEnvConfig(void) { ReloadEnvConfig(); AlgoPluginReload(); return HCCL_SUCCESS; }
HcclResult HcclAlgoPluginQueryAlgs(const char* opName, char* buf, uint32_t bufLen, uint32_t* count) { return AlgoPluginQueryAlgs(opName, buf, bufLen, count); }
const char* HcclGetErrorString(HcclResult code) { return ResultString(code); }

HcclResult HcclGetRootInfo(HcclRootInfo* rootInfo)
{
    CHK_PTR_NULL(rootInfo);
    return BootstrapCreateRoot(rootInfo);
}

HcclResult HcclCommInitRootInfoConfig(uint32_t nRanks, const HcclRootInfo* rootInfo, uint32_t rank, const HcclCommConfig* config,
                                      HcclComm* comm)
{
    CHK_PTR_NULL(rootInfo);
    CHK_PTR_NULL(comm);
    if (nRanks == 0 || rank >= nRanks) { HCCL_ERROR("HcclCommInitRootInfo: rank %u out of range for %u ranks", rank, nRanks); return HCCL_E_PARA; }
    CommImpl* c = new CommImpl();
    HcclResult r = c->Init(*rootInfo, (int)nRanks, (int)rank, config);
    if (r != HCCL_SUCCESS) { delete c; return r; }
    *comm = c;
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitRootInfo(uint32_t nRanks, const HcclRootInfo* rootInfo, uint32_t rank, HcclComm* comm)
{
    return HcclCommInitRootInfoConfig(nRanks, rootInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitClusterInfoConfig(const char* clusterInfo, uint32_t rank, const HcclCommConfig* config, HcclComm* comm)
{
    CHK_PTR_NULL(clusterInfo);
    CHK_PTR_NULL(comm);
    RankTable table;
    CHK_RET(LoadRankTable(clusterInfo, &table));
    if (rank >= table.ranks.size()) { HCCL_ERROR("rank %u is not in the rank table (%zu ranks)", rank, table.ranks.size()); return HCCL_E_PARA; }
    int dev = table.ranks[rank].deviceId;
    if (dev >= 0) CHK_CUDA(cudaSetDevice(dev));
    // The rank table fixes the rendezvous address; rank 0 hosts the relay.  The id is derived from the table so that
    // all ranks agree without any exchange.
    HcclRootInfo info;
    memset(&info, 0, sizeof(info));
    if (rank == 0) {
        CHK_RET(BootstrapCreateRootAt(table.rootIp, table.rootPort, table.Fingerprint(), &info));
    } else {
        RootInfoPayload* p = reinterpret_cast<RootInfoPayload*>(info.internal);
        p->magic = kRootInfoMagic; p->version = 1; p->port = table.rootPort; p->uniqueId = table.Fingerprint();
        snprintf(p->ip, sizeof(p->ip), "%s", table.rootIp.c_str());
    }
    return HcclCommInitRootInfoConfig((uint32_t)table.ranks.size(), &info, rank, config, comm);
}

HcclResult HcclCommInitClusterInfo(const char* clusterInfo, uint32_t rank, HcclComm* comm)
{
    return HcclCommInitClusterInfoConfig(clusterInfo, rank, nullptr, comm);
}

HcclResult HcclCommInitEmulated(uint32_t nRanks, const HcclCommConfig* config, HcclComm* comms)
{
    CHK_PTR_NULL(comms);
    std::vector<CommImpl*> v;
    CHK_RET(EmuGroup::Create((int)nRanks, config, &v));
    for (uint32_t i = 0; i < nRanks; ++i) comms[i] = v[i];
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitHostSim(uint32_t nRanks, const char* topoJson, const HcclCommConfig* config, HcclComm* comms)
{
    CHK_PTR_NULL(comms);
    std::vector<CommImpl*> v(nRanks, nullptr);
    CHK_RET(HostWorldCreate(nRanks, topoJson, config, v.data()));
    for (uint32_t i = 0; i < nRanks; ++i) comms[i] = v[i];
    return HCCL_SUCCESS;
}

HcclResult HcclCommInitAll(uint32_t ndev, const int32_t* devices, HcclComm* comms)
{
    CHK_PTR_NULL(devices);
    CHK_PTR_NULL(comms);
    if (ndev == 0) return HCCL_E_PARA;
    bool allHost = true, allSame = true;
    for (uint32_t i = 0; i < ndev; ++i) { allHost = allHost && devices[i] < 0; allSame = allSame && devices[i] == devices[0]; }
    if (allHost) return HcclCommInitHostSim(ndev, nullptr, nullptr, comms);
    if ((allSame && ndev > 1) || GetEnvConfig().emulate) {
        CHK_CUDA(cudaSetDevice(devices[0]));
        return HcclCommInitEmulated(ndev, nullptr, comms);
    }
    // one thread per device runs the ordinary root-info initialisation
    HcclRootInfo info;
    CHK_RET(HcclGetRootInfo(&info));
    std::vector<HcclResult> res(ndev, HCCL_SUCCESS);
    std::vector<std::thread> th;
    for (uint32_t i = 0; i < ndev; ++i) {
        th.emplace_back([&, i] {
            if (cudaSetDevice(devices[i]) != cudaSuccess) { res[i] = HCCL_E_RUNTIME; return; }
            res[i] = HcclCommInitRootInfo(ndev, &info, i, &comms[i]);
        });
    }
    for (auto& t : th) t.join();
    for (HcclResult r : res) if (r != HCCL_SUCCESS) return r;
    return HCCL_SUCCESS;
}

HcclResult HcclCommDestroy(HcclComm comm)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    HcclResult r = c->Destroy();
    delete c;
    return r;
}

HcclResult HcclGetRankSize(HcclComm comm, uint32_t* n) { CHK_PTR_NULL(comm); CHK_PTR_NULL(n); *n = (uint32_t) static_cast<CommImpl*>(comm)->nRanks; return HCCL_SUCCESS; }
HcclResult HcclGetRankId(HcclComm comm, uint32_t* r) { CHK_PTR_NULL(comm); CHK_PTR_NULL(r); *r = (uint32_t) static_cast<CommImpl*>(comm)->rank; return HCCL_SUCCESS; }
HcclResult HcclGetCommName(HcclComm comm, char* name)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(name);
    snprintf(name, HCCL_COMM_CONFIG_NAME_MAX, "%s", static_cast<CommImpl*>(comm)->name.c_str());
    return HCCL_SUCCESS;
}
HcclResult HcclCommGetStatus(HcclComm comm, HcclCommStatus* st)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(st);
    CommImpl* c = static_cast<CommImpl*>(comm);
    HcclResult e;
    c->PollAsyncError(&e);
    *st = (HcclCommStatus)c->status_.load();
    return HCCL_SUCCESS;
}
HcclResult HcclCommSuspend(HcclComm comm) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->Suspend(); }
HcclResult HcclCommResume(HcclComm comm) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->Resume(); }
HcclResult HcclCommGetAsyncError(HcclComm comm, HcclResult* e) { CHK_PTR_NULL(comm); CHK_PTR_NULL(e); return static_cast<CommImpl*>(comm)->PollAsyncError(e); }

HcclResult HcclGetHcclBuffer(HcclComm comm, void** buffer, uint64_t* size)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(buffer); CHK_PTR_NULL(size);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (c->hostComm) return HCCL_E_NOT_SUPPORT;
    *buffer = c->StageBase(c->rank);
    *size = c->layout().dataBytes;
    return HCCL_SUCCESS;
}

HcclResult HcclMemAlloc(HcclComm comm, uint64_t size, void** p) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->MemAlloc(size, p); }
HcclResult HcclMemFree(HcclComm comm, void* p) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->MemFree(p); }
HcclResult HcclCommRegister(HcclComm comm, void* devPtr, uint64_t size) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->RegisterBuffer(devPtr, size); }
HcclResult HcclCommDeregister(HcclComm comm, void* devPtr) { CHK_PTR_NULL(comm); return static_cast<CommImpl*>(comm)->DeregisterBuffer(devPtr); }
HcclResult HcclCommSymWinGet(HcclComm comm, const void* localPtr, uint32_t peerRank, void** peerPtr)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(peerPtr);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (peerRank >= (uint32_t)c->nRanks) return HCCL_E_PARA;
    const char* peers[kMaxDevRanks];
    if (!c->Lookup(localPtr, 1, peers, nullptr)) return HCCL_E_NOT_FOUND;
    *peerPtr = const_cast<char*>(peers[peerRank]);
    return HCCL_SUCCESS;
}
HcclResult HcclCommSymWinGetMulticast(HcclComm comm, const void* localPtr, void** mcPtr)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(mcPtr);
    CommImpl* c = static_cast<CommImpl*>(comm);
    const char* peers[kMaxDevRanks];
    const char* mc = nullptr;
    if (!c->Lookup(localPtr, 1, peers, &mc)) return HCCL_E_NOT_FOUND;
    *mcPtr = const_cast<char*>(mc);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- extensions
HcclResult HcclGetLastAlgName(HcclComm comm, char* name, uint32_t cap)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(name);
    std::vector<uint8_t> b;
    std::string s;
    if (static_cast<CommImpl*>(comm)->ctx.Get("last_alg", &b)) s.assign(b.begin(), b.end());
    snprintf(name, cap, "%s", s.c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclSelectorExplain(HcclComm comm, HcclCMDType op, uint64_t count, HcclDataType dt, HcclReduceOp rop, int registered, char* text, uint32_t cap)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(text);
    CommImpl* c = static_cast<CommImpl*>(comm);
    OpDesc d;
    d.op = op; d.dtype = dt; d.redOp = rop; d.nRanks = (uint32_t)c->nRanks; d.det = c->cfg.deterministic; d.engine = c->cfg.engine;
    uint64_t es = 1;
    switch (dt) { case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: es = 4; break; case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: case HCCL_DATA_TYPE_INT16: es = 2; break;
                  case HCCL_DATA_TYPE_FP64: case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: es = 8; break; default: es = 1; }
    d.bytes = count * es;
    if (op == HCCL_CMD_ALLGATHER || op == HCCL_CMD_REDUCE_SCATTER || op == HCCL_CMD_SCATTER || op == HCCL_CMD_ALLTOALL) d.bytes *= (uint64_t)c->nRanks;
    d.inRegistered = d.outRegistered = registered != 0;
    d.stageInBytes = c->layout().inBytes;
    d.inMulticast = d.outMulticast = registered != 0 && c->nvls();      // "registered" here means HcclMemAlloc memory
    Selection sel;
    HcclResult r = SelectAlgorithm(*c->selector, *c->topo, GetEnvConfig(), d, c->name, comm, c->cfg.bufferBytes, &sel);
    std::string s = (sel.alg ? "selected " + sel.alg->name + "\n" : std::string("selected none\n")) + FormatCostTable(sel);
    snprintf(text, cap, "%s", s.c_str());
    return r;
}

}  // extern "C"

namespace {
// What a communicator is to the resource query: everything the answer depends on.  Filled from a live communicator
// (online) or from a description of the box (offline: no device, no communicator).
struct ResQueryCtx {
    const TopoInfo* topo;
    SelectorState* selector;
    StageLayout layout;
    uint64_t bufferBytes;
    int nRanks, maxBlocks;
    HcclCommEngine engine;
    Deterministic det;
    bool nvls, host;
    std::string name;
    HcclComm comm;
};

HcclResult CalcOpRes(const ResQueryCtx& q, HcclCMDType op, uint64_t count, HcclDataType dt, HcclReduceOp rop, int registered, HcclOpResource* res)
{
    memset(res, 0, sizeof(*res));
    res->streams = 1;
    OpDesc d;
    d.op = op; d.dtype = dt; d.redOp = rop; d.nRanks = (uint32_t)q.nRanks; d.det = q.det;
    d.engine = q.host ? HCCL_ENGINE_HOSTCPU : q.engine;
    const uint64_t es = DataTypeSize(dt);
    if (es == 0) return HCCL_E_PARA;
    const uint64_t P = (uint64_t)q.nRanks;
    const bool perRank = op == HCCL_CMD_ALLGATHER || op == HCCL_CMD_REDUCE_SCATTER || op == HCCL_CMD_SCATTER || op == HCCL_CMD_ALLTOALL;
    d.bytes = count * es * (perRank ? P : 1);
    d.inRegistered = d.outRegistered = registered != 0;
    d.stageInBytes = q.layout.inBytes;
    d.inMulticast = d.outMulticast = registered != 0 && q.nvls;      // "registered" here means HcclMemAlloc memory
    Selection sel;
    CHK_RET(SelectAlgorithm(*q.selector, *q.topo, GetEnvConfig(), d, q.name, q.comm, q.bufferBytes, &sel));
    snprintf(res->algName, sizeof(res->algName), "%s", sel.alg->name.c_str());
    res->engine = (uint32_t)sel.alg->engine;
    if (q.host || q.nRanks == 1) { res->blocks = 0; res->launches = q.nRanks == 1 ? 0 : 1; return HCCL_SUCCESS; }
    // mirror of the sole executor's loop bound: staged inputs go through the stage-in region, two-shot results through the exchange region
    const StageLayout& L = q.layout;
    const bool ll = sel.alg->devAlg == DALG_AR_LL || sel.alg->devAlg == DALG_AG_LL;
    uint64_t staged = (registered || ll) ? 0 : d.bytes;
    if (op == HCCL_CMD_ALLGATHER && !registered) staged = d.bytes / P;
    uint64_t limit = registered ? ~0ull : (perRank && op != HCCL_CMD_ALLGATHER ? L.inBytes / P * P : L.inBytes);
    if (sel.alg->devAlg == DALG_AR_TWOSHOT || sel.alg->devAlg == DALG_AR_NVLS || sel.alg->devAlg == DALG_BCAST_TWOSHOT || sel.alg->devAlg == DALG_REDUCE_TWOSHOT)
        limit = std::min<uint64_t>(limit, L.xchBytes);
    // push forms: one landing copy (half of the stage-in region) holds a launch's blocks
    if (sel.alg->devAlg == DALG_AR_PUSH_TWOSHOT) limit = std::min<uint64_t>(L.inBytes / 2 / 128 * 128 - 16 * P, L.xchBytes);
    if (sel.alg->devAlg == DALG_RS_PUSH) limit = L.inBytes / 2 / P / 128 * 128 * P;
    res->launches = (uint32_t)std::max<uint64_t>(1, limit == ~0ull || d.bytes == 0 ? 1 : (d.bytes + limit - 1) / limit);
    res->scratchBytes = std::min<uint64_t>(staged, limit == ~0ull ? staged : limit);
    const uint64_t perLaunch = d.bytes / res->launches;
    uint64_t traffic = perLaunch;
    if (sel.alg->devAlg == DALG_AR_TWOSHOT || sel.alg->devAlg == DALG_AR_NVLS || sel.alg->devAlg == DALG_AR_PUSH_TWOSHOT) traffic = perLaunch / P * 2 + 1;
    if (sel.alg->devAlg == DALG_RS_PUSH) traffic = perLaunch / P + 1;
    uint64_t nb = ll ? std::min<uint64_t>((perLaunch / (op == HCCL_CMD_ALLGATHER ? P : 1) + 8191) / 8192, 8) : (traffic + (128u << 10) - 1) / (128u << 10);
    res->blocks = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(nb, (uint64_t)q.maxBlocks));
    return HCCL_SUCCESS;
}
}  // namespace

extern "C" {

HcclResult HcclCalcOpResource(HcclComm comm, HcclCMDType op, uint64_t count, HcclDataType dt, HcclReduceOp rop, int registered, HcclOpResource* res)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(res);
    CommImpl* c = static_cast<CommImpl*>(comm);
    const ResQueryCtx q{c->topo.get(), c->selector.get(), c->layout(), c->cfg.bufferBytes, c->nRanks, c->MaxBlocks(), c->cfg.engine, c->cfg.deterministic,
                        c->nvls(), c->hostComm != nullptr, c->name, comm};
    return CalcOpRes(q, op, count, dt, rop, registered, res);
}

// The same answer without a communicator or a device: one NVSwitch box of nRanks GPUs, a staging slab of bufferBytes
// (0 = the default), the environment's engine and determinism settings.  (The reference sizes a graph node's resources
// before any communicator exists: HcclCalcOpResOfflineGraphMode, interface_graph_mode/calc_resource_graph_mode.cc.)
HcclResult HcclCalcOpResOfflineGraphMode(uint32_t nRanks, int nvls, uint64_t bufferBytes, HcclCMDType op, uint64_t count, HcclDataType dt,
                                         HcclReduceOp rop, int registered, HcclOpResource* res)
{
    CHK_PTR_NULL(res);
    if (nRanks < 1 || nRanks > (uint32_t)kMaxDevRanks) return HCCL_E_PARA;
    EnsureAlgorithmsRegistered();
    EffectiveConfig eff;
    CHK_RET(MergeConfig(GetEnvConfig(), nullptr, &eff));
    if (bufferBytes) eff.bufferBytes = bufferBytes;
    const TopoInfo topo = SyntheticNvswitchBox(nRanks, nvls != 0, GlobalLinkModel().p2pGBs);
    SelectorState st;
    int maxBlocks = eff.maxBlocks ? (int)eff.maxBlocks : 128;
    if (maxBlocks > kMaxBlocks) maxBlocks = kMaxBlocks;
    const ResQueryCtx q{&topo, &st, MakeStageLayout(eff.bufferBytes, (int)nRanks), eff.bufferBytes, (int)nRanks, maxBlocks, eff.engine, eff.deterministic,
                        nvls != 0, false, "offline", nullptr};
    return CalcOpRes(q, op, count, dt, rop, registered, res);
}

uint32_t HcclAlgRegistryCount(void)
{
    EnsureAlgorithmsRegistered();
    return (uint32_t)AlgRegistry::Instance().All().size();
}
HcclResult HcclAlgRegistryEntry(uint32_t i, char* name, uint32_t cap, HcclCMDType* op, HcclCommEngine* engine)
{
    EnsureAlgorithmsRegistered();
    const auto& all = AlgRegistry::Instance().All();
    if (i >= all.size()) return HCCL_E_PARA;
    if (name) snprintf(name, cap, "%s", all[i].name.c_str());
    if (op) *op = all[i].op;
    if (engine) *engine = all[i].engine;
    return HCCL_SUCCESS;
}

HcclResult HcclProfilingSetLevel(int level) { SetProfilingLevel(level); return HCCL_SUCCESS; }
HcclResult HcclProfilingDump(char* text, uint32_t cap)
{
    CHK_PTR_NULL(text);
    std::ostringstream os;
    os << "seq,op,alg,comm,rank,rankSize,dtype,count,bytes,host_us,device_us\n";
    for (const ProfRecord& r : ProfilingSnapshot())
        os << r.seq << "," << r.op << "," << r.alg << "," << r.comm << "," << r.rank << "," << r.rankSize << "," << r.dtype << "," << r.count << ","
           << r.bytes << "," << r.hostSubmitUs << "," << r.deviceUs << "\n";
    snprintf(text, cap, "%s", os.str().c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclTestLaunchUnsignalledWait(HcclComm comm, hcclStream_t stream)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (c->hostComm) return HCCL_E_NOT_SUPPORT;
    CollArgs a;
    memset(&a, 0, sizeof(a));
    LaunchTarget t = c->Target((cudaStream_t)stream);
    t.emu = nullptr;   // a single rank waits on its own: no cooperative launch needed
    return LaunchCollective(t, DALG_TEST_WAIT, HCCL_DATA_TYPE_INT8, a, 1);
}
HcclResult HcclTestInjectBootstrapFailure(HcclComm comm)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->bs) return HCCL_E_NOT_SUPPORT;
    c->bs->InjectFailureOnce();
    return HCCL_SUCCESS;
}
HcclResult HcclGetPlanCacheStats(HcclComm comm, uint64_t* hits, uint64_t* misses, uint64_t* entries)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->plans) return HCCL_E_NOT_SUPPORT;
    if (hits) *hits = c->plans->hits();
    if (misses) *misses = c->plans->misses();
    if (entries) *entries = c->plans->size();
    return HCCL_SUCCESS;
}
HcclResult HcclSetLinkModel(double p2p, double nvls, double copy, double launch, double barrier, double ll)
{
    LinkModel& m = GlobalLinkModel();
    if (p2p > 0) m.p2pGBs = p2p;
    if (nvls > 0) m.nvlsGBs = nvls;
    if (copy > 0) { m.localCopyGBs = copy; m.localReduceGBs = copy; }
    if (launch >= 0) m.launchUs = launch;
    if (barrier >= 0) m.barrierUs = barrier;
    if (ll >= 0) m.llHopUs = ll;
    return HCCL_SUCCESS;
}

}  // extern "C"
