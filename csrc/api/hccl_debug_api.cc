// Text renderings of pure functions (step tables, HCCL_ALGO / environment parsing, cost formula) for unit tests.
#include <cstring>
#include <map>
#include <sstream>
#include "../algo/step_tables.h"
#include "../core/bootstrap.h"
#include "../core/config.h"
#include "../core/log.h"
#include "../core/plan_cache.h"
#include "../cpu/host_tree.h"
#include "../select/auto_selector.h"
#include "../select/selector.h"
#include "hccl/hccl_ext.h"
#include "ranktable.h"

using namespace hccl;

namespace {
template <class V>
std::string Join(const V& v)
{
    std::ostringstream os;
    bool first = true;
    for (auto x : v) { os << (first ? "" : ",") << x; first = false; }
    return os.str();
}
}  // namespace

extern "C" {

HcclResult HcclDebugStepTable(const char* kind, uint32_t p, uint32_t rank, const char* arg, char* text, uint32_t cap)
{
    CHK_PTR_NULL(kind); CHK_PTR_NULL(text);
    std::ostringstream os;
    const std::string k(kind);
    if (k == "nhr_rs" || k == "nhr_ag") {
        for (const NhrStep& s : (k == "nhr_rs" ? NhrReduceScatterSteps(p, rank) : NhrAllGatherSteps(p, rank)))
            os << "step " << s.step << " to " << s.sendTo << " from " << s.recvFrom << " tx [" << Join(s.txSlices) << "] rx [" << Join(s.rxSlices) << "]\n";
    } else if (k == "rhd_rs" || k == "rhd_ag") {
        const RhdInfo i = RhdPart1(p, rank);
        if (!i.merged)
            for (const RhdStep& s : (k == "rhd_rs" ? RhdReduceScatterSteps(p, i.vrank) : RhdAllGatherSteps(p, i.vrank)))
                os << "peer " << RhdVirtualToReal(p, s.peerVirtual) << " send [" << s.sendUnitBegin << "," << s.sendUnitEnd << ") keep [" << s.keepUnitBegin << ","
                   << s.keepUnitEnd << ")\n";
    } else if (k == "rhd_info") {
        const RhdInfo i = RhdPart1(p, rank);
        os << "P " << i.P << " r " << i.r << " steps " << i.steps << " merged " << i.merged << " representative " << i.representative << " partner "
           << i.partner << " vrank " << i.vrank << " sigma " << RhdSigma(p, rank) << "\n";
    } else if (k == "ring_rs" || k == "ring_ag") {
        for (const RingStep& s : (k == "ring_rs" ? RingReduceScatterSteps(p, rank) : RingAllGatherSteps(p, rank))) os << "send " << s.sendSlice << " recv " << s.recvSlice << "\n";
    } else if (k == "pairwise") {
        for (const PairwiseStep& s : PairwiseSteps(p, rank)) os << "to " << s.sendTo << " from " << s.recvFrom << "\n";
    } else if (k == "bruck_ag") {
        for (const BruckStep& s : BruckAllGatherSteps(p, rank))
            os << "to " << s.sendTo << " from " << s.recvFrom << " send " << s.firstSendBlock << " recv " << s.firstRecvBlock << " n " << s.nBlocks << "\n";
    } else if (k == "nb_scatter") {
        for (const TreeScatterStep& s : BinomialScatterSteps(p, rank))
            os << (s.sends ? "send" : s.receives ? "recv" : "idle") << " peer " << s.peer << " first " << s.firstBlock << " n " << s.nBlocks << "\n";
    } else if (k == "bw_split") {
        // arg = "count,bwA,bwB,align"
        unsigned long long count = 0, align = 1;
        double a = 0, b = 0;
        if (!arg || sscanf(arg, "%llu,%lf,%lf,%llu", &count, &a, &b, &align) != 4) return HCCL_E_PARA;
        os << BandwidthSplit(count, a, b, align) << "\n";
    } else if (k == "pipeline") {
        // p = stages, rank = steps
        for (const PipeSlot& s : PipelineSchedule(p, rank)) os << "t " << s.time << " stage " << s.stage << " step " << s.step << "\n";
    } else if (k == "ifname") {
        // arg = "rule|name,name,...": which interface a rule of HCCL_SOCKET_IFNAME selects
        const std::string a = arg ? arg : "";
        const size_t bar = a.find('|');
        std::vector<std::string> names;
        std::stringstream ns(bar == std::string::npos ? std::string() : a.substr(bar + 1));
        for (std::string n; std::getline(ns, n, ',');) names.push_back(n);
        const int i = MatchInterfaceRule(a.substr(0, bar), names);
        os << (i < 0 ? std::string("none") : names[(size_t)i]) << "\n";
    } else if (k == "parse_tree") {
        std::unique_ptr<AlgoTreeNode> tree;
        std::string err;
        if (!ParseAlgoTree(arg ? arg : "", &tree, &err)) os << "error: " << err << "\n";
        else os << AlgoTreeText(*tree) << " queues " << AlgoTreeQueues(*tree) << " levels " << AlgoTreeMinLevels(*tree) << "\n";
    } else if (k == "threshold") {
        // p = ranks, rank = topology levels, arg = "op,bytes,host,nvls,strict"
        ThresholdInput in;
        int op = 0, host = 0, nvls = 0, strict = 0;
        unsigned long long bytes = 0;
        if (!arg || sscanf(arg, "%d,%llu,%d,%d,%d", &op, &bytes, &host, &nvls, &strict) != 5) return HCCL_E_PARA;
        in.op = (HcclCMDType)op; in.bytes = bytes; in.nRanks = p; in.levels = rank; in.hostEngine = host; in.nvls = nvls; in.strictOrder = strict;
        os << ThresholdSelect(in) << "\n";
    } else if (k == "rank_table") {
        // arg = rank-table JSON text or a file path
        RankTable t;
        const HcclResult r = LoadRankTable(arg ? arg : "", &t);
        if (r != HCCL_SUCCESS) os << "error: " << ResultString(r) << "\n";
        else {
            os << "ranks " << t.ranks.size() << " servers";
            for (uint32_t n : t.serverSizes) os << " " << n;
            os << " root " << t.rootIp << ":" << t.rootPort << " fingerprint " << t.Fingerprint() << "\n";
            for (const RankTableEntry& e : t.ranks) os << "rank " << e.rankId << " server " << e.serverId << " device " << e.deviceId << " ip " << e.deviceIp << "\n";
        }
    } else if (k == "plan_cache") {
        // p = keys to insert (bytes = 1..p); key 1 is looked up again after every 1000 inserts, so it stays recent.
        // Reports the size, whether key 1 / key 2 / the newest key are present, and a lookup under another generation.
        PlanCache cache;
        Plan plan;
        for (uint32_t i = 1; i <= p; ++i) {
            PlanKey key{2, 4, 0, 0, i, 0, 7};
            plan.algIndex = (int)i;
            cache.Insert(key, plan);
            if (i % 1000 == 0) { PlanKey first{2, 4, 0, 0, 1, 0, 7}; cache.Find(first, &plan); }
        }
        Plan got;
        const bool has1 = cache.Find(PlanKey{2, 4, 0, 0, 1, 0, 7}, &got);
        const bool has2 = cache.Find(PlanKey{2, 4, 0, 0, 2, 0, 7}, &got);
        const bool hasLast = cache.Find(PlanKey{2, 4, 0, 0, p, 0, 7}, &got);
        const int lastAlg = hasLast ? got.algIndex : -1;
        const bool otherGen = cache.Find(PlanKey{2, 4, 0, 0, p, 0, 8}, &got);
        os << "capacity " << PlanCache::kCapacity << " size " << cache.size() << " key1 " << has1 << " key2 " << has2 << " newest " << hasLast << " alg " << lastAlg
           << " other_generation " << otherGen << " hits " << cache.hits() << " misses " << cache.misses() << "\n";
    } else if (k == "fold") {
        for (auto& pr : DeterministicFoldOrder(p)) os << pr.first << "+=" << pr.second << "\n";
    } else if (k == "parse_algo") {
        AlgoConfig cfg;
        std::string err;
        if (!ParseHcclAlgo(arg ? arg : "", &cfg, &err)) os << "error: " << err << "\n";
        else {
            auto dump = [&](const char* name, const AlgoLevelConfig& l) {
                os << name << ":";
                for (int i = 0; i < kAlgoLevels; ++i) os << " " << AlgoTypeName(l.level[i]);
                os << "\n";
            };
            dump("global", cfg.global);
            for (auto& kv : cfg.perOp) dump(("op" + std::to_string((int)kv.first)).c_str(), kv.second);
        }
    } else {
        return HCCL_E_PARA;
    }
    snprintf(text, cap, "%s", os.str().c_str());
    return HCCL_SUCCESS;
}

// Selection for a synthetic one-box NVSwitch topology (no device needed): what the selector would run for one call on
// `nRanks` GPUs with or without switch reduction, on symmetric (registered != 0) or plain buffers, under a determinism
// level (0 off, 1 on, 2 strict).  Same text as HcclSelectorExplain.
HcclResult HcclDebugExplainDevice(uint32_t nRanks, int nvls, HcclCMDType op, uint64_t bytes, HcclDataType dt, HcclReduceOp rop, int registered,
                                  int deterministic, char* text, uint32_t cap)
{
    CHK_PTR_NULL(text);
    if (nRanks < 2 || nRanks > 8) return HCCL_E_PARA;
    const TopoInfo topo = SyntheticNvswitchBox(nRanks, nvls != 0, GlobalLinkModel().p2pGBs);
    OpDesc d;
    d.op = op; d.dtype = dt; d.redOp = rop; d.nRanks = nRanks; d.bytes = bytes;
    d.det = deterministic == 2 ? Deterministic::STRICT : deterministic == 1 ? Deterministic::ON : Deterministic::OFF;
    d.inRegistered = d.outRegistered = registered != 0;
    d.inMulticast = d.outMulticast = registered != 0 && nvls != 0;
    d.stageInBytes = 100ull << 20;          // the stage-in region of the default 256 MiB slab
    SelectorState st;
    Selection sel;
    const HcclResult r = SelectAlgorithm(st, topo, GetEnvConfig(), d, "synthetic", nullptr, 256ull << 20, &sel);
    const std::string s = (sel.alg ? "selected " + sel.alg->name + "\n" : std::string("selected none\n")) + FormatCostTable(sel);
    snprintf(text, cap, "%s", s.c_str());
    return r;
}

// ---- the bootstrap on its own (no device): connection, all-gather, barrier, agreement, failure paths
HcclResult HcclDebugBootstrapConnect(const HcclRootInfo* info, uint32_t rank, uint32_t nRanks, uint32_t timeoutS, void** handle)
{
    CHK_PTR_NULL(info); CHK_PTR_NULL(handle);
    auto* b = new Bootstrap();
    const HcclResult r = b->Connect(*info, (int)rank, (int)nRanks, timeoutS);
    if (r != HCCL_SUCCESS) { delete b; *handle = nullptr; return r; }
    *handle = b;
    return HCCL_SUCCESS;
}
HcclResult HcclDebugBootstrapAllGather(void* handle, const void* send, void* recv, uint64_t bytesPerRank)
{
    CHK_PTR_NULL(handle); CHK_PTR_NULL(send); CHK_PTR_NULL(recv);
    return static_cast<Bootstrap*>(handle)->AllGather(send, recv, (size_t)bytesPerRank);
}
HcclResult HcclDebugBootstrapBarrier(void* handle)
{
    CHK_PTR_NULL(handle);
    return static_cast<Bootstrap*>(handle)->Barrier();
}
HcclResult HcclDebugBootstrapAgree(void* handle, int ok, int* all)
{
    CHK_PTR_NULL(handle); CHK_PTR_NULL(all);
    bool a = false;
    const HcclResult r = static_cast<Bootstrap*>(handle)->AgreeAll(ok != 0, &a);
    *all = a ? 1 : 0;
    return r;
}
HcclResult HcclDebugBootstrapInjectFailure(void* handle)
{
    CHK_PTR_NULL(handle);
    static_cast<Bootstrap*>(handle)->InjectFailureOnce();
    return HCCL_SUCCESS;
}
HcclResult HcclDebugBootstrapClose(void* handle)
{
    CHK_PTR_NULL(handle);
    Bootstrap* b = static_cast<Bootstrap*>(handle);
    b->Close();
    delete b;
    return HCCL_SUCCESS;
}

HcclResult HcclDiagnoseDump(char* text, uint32_t capacity)
{
    CHK_PTR_NULL(text);
    if (capacity == 0) return HCCL_E_PARA;
    const std::string all = DiagnoseDump();
    // keep the newest lines when the buffer is short
    const size_t skip = all.size() + 1 > capacity ? all.size() + 1 - capacity : 0;
    snprintf(text, capacity, "%s", all.c_str() + skip);
    return HCCL_SUCCESS;
}

HcclResult HcclDebugParseEnv(const char* settings, char* text, uint32_t cap)
{
    CHK_PTR_NULL(settings); CHK_PTR_NULL(text);
    std::map<std::string, std::string> vars;
    std::istringstream is(settings);
    std::string line;
    while (std::getline(is, line)) {
        size_t eq = line.find('=');
        if (eq != std::string::npos) vars[line.substr(0, eq)] = line.substr(eq + 1);
    }
    EnvConfig c = ParseEnvConfig([&](const char* n) -> const char* {
        auto it = vars.find(n);
        return it == vars.end() ? nullptr : it->second.c_str();
    });
    EffectiveConfig eff;
    MergeConfig(c, nullptr, &eff);
    TimeoutChain tc = DeriveTimeouts(eff.execTimeoutNs);
    std::ostringstream os;
    os << "engine=" << (int)c.expansionMode << " planCache=" << c.planCacheEnable << " deterministic=" << (int)c.deterministic << " execTimeoutS=" << c.execTimeoutS
       << " retryL1=" << c.retryL1 << " retryL2=" << c.retryL2 << " retryMaxCnt=" << c.retryMaxCnt << " stuck=" << c.dfs.stuckDetection << " heartbeat="
       << c.dfs.clusterHeartbeat << " inconsistent=" << c.dfs.inconsistentCheck << " faultTime=" << c.dfs.connectionFaultDetectionTimeS << " debugMask="
       << c.debugConfigMask << " entryLog=" << c.entryLog << " bufferMiB=" << c.bufferSizeMiB << " ifIp=" << c.ifIp << " basePort=" << c.ifBasePort
       << " connectTimeoutS=" << c.connectTimeoutS << " nvls=" << c.nvlsEnable << " maxBlocks=" << c.maxBlocks << " split=" << Join(c.splitRatio)
       << " algoSpecified=" << c.algo.global.specified << " perOp=" << c.algo.perOp.size() << "\n";
    os << "effective bufferBytes=" << eff.bufferBytes << " execTimeoutNs=" << eff.execTimeoutNs << " waitNs=" << tc.waitNs << " fullNs=" << tc.fullNs << " kernelNs="
       << tc.kernelNs << " hostNotifyNs=" << tc.hostNotifyNs << "\n";
    os << "bootstrap ifname=" << c.socketIfname << " ipv6=" << c.socketIpv6 << " whitelistDisable=" << c.whitelistDisable << " whitelistFile=" << c.whitelistFile
       << " portAuto=" << c.hostPortAuto << " ports=";
    for (auto& r : c.hostPortRanges) os << r.first << "-" << r.second << ";";
    os << " notApplicable=" << c.notApplicable.size() << "\n";
    for (auto& e : c.errors) os << "rejected: " << e << "\n";
    snprintf(text, cap, "%s", os.str().c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclLoadLinkModel(const char* path, char* error, uint32_t cap)
{
    CHK_PTR_NULL(path);
    std::string err;
    const bool ok = LoadLinkModelFile(path, &err);
    if (error && cap) snprintf(error, cap, "%s", err.c_str());
    return ok ? HCCL_SUCCESS : HCCL_E_PARA;
}
double HcclDebugLinkUtilisation(int netType, double bytes, uint32_t nRanks) { return LinkUtilisation((NetType)netType, bytes, HCCL_ENGINE_P2P, (int)nRanks); }

double HcclDebugEvalCost(double A, double B, double C, double D, int netType, double ratio, double bytes)
{
    CostCoeff c;
    c.A = A; c.B = B; c.C = C; c.D = D; c.net = (NetType)netType; c.ratio = ratio;
    return EvalCost({c}, CostAgg::SUM, bytes, HCCL_ENGINE_P2P);
}

}  // extern "C"
