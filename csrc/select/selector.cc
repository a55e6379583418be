#include "selector.h"
#include "auto_selector.h"
#include <atomic>
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <mutex>
#include <sstream>
#include "../core/json.h"
#include "../core/log.h"

namespace hccl {

// Bits of Flags() that describe THIS rank's buffers; the rest is communicator-wide.
constexpr uint32_t kCapabilityBits = 1u | 2u | 4u | (1u << 20) | (1u << 21);
constexpr uint32_t kInPlaceBit = 8u;

uint32_t OpDesc::CombineFlags(uint32_t a, uint32_t b)
{
    // a capability holds for the call only when every rank has it; one rank working in place makes the call in place
    return (a & b & kCapabilityBits) | ((a | b) & kInPlaceBit) | (a & ~(kCapabilityBits | kInPlaceBit));
}

void OpDesc::ApplyFlags(uint32_t f)
{
    inRegistered = (f & 1u) != 0;
    outRegistered = (f & 2u) != 0;
    aligned16 = (f & 4u) != 0;
    inPlace = (f & 8u) != 0;
    inMulticast = (f & (1u << 20)) != 0;
    outMulticast = (f & (1u << 21)) != 0;
}

uint32_t OpDesc::Flags() const
{
    return (inRegistered ? 1u : 0u) | (outRegistered ? 2u : 0u) | (aligned16 ? 4u : 0u) | (inPlace ? 8u : 0u) | (inMulticast ? (1u << 20) : 0u) |
           (outMulticast ? (1u << 21) : 0u) |
           (isMc2 ? 16u : 0u) | ((uint32_t)det << 5) | ((uint32_t)engine << 8) | (castScale ? (1u << 22) : 0u);
}

// ------------------------------------------------------------------ registry
AlgRegistry& AlgRegistry::Instance()
{
    static AlgRegistry r;
    return r;
}
int AlgRegistry::Register(AlgEntry e)
{
    for (auto& a : algs_)
        if (a.op == e.op && a.name == e.name) {
            HCCL_WARNING("algorithm %s registered twice for op %d: second registration ignored", e.name.c_str(), (int)e.op);
            return -1;
        }
    algs_.push_back(std::move(e));
    return (int)algs_.size() - 1;
}
const AlgEntry* AlgRegistry::Find(HcclCMDType op, const std::string& name) const
{
    int i = IndexOf(op, name);
    return i < 0 ? nullptr : &algs_[(size_t)i];
}
int AlgRegistry::IndexOf(HcclCMDType op, const std::string& name) const
{
    for (size_t i = 0; i < algs_.size(); ++i)
        if (algs_[i].op == op && algs_[i].name == name) return (int)i;
    return -1;
}
std::vector<int> AlgRegistry::ForOp(HcclCMDType op) const
{
    std::vector<int> v;
    for (size_t i = 0; i < algs_.size(); ++i)
        if (algs_[i].op == op) v.push_back((int)i);
    return v;
}

bool MapAlgName(const AlgEntry& e, AlgNameDims* out)
{
    switch (e.engine) {
        case HCCL_ENGINE_P2P: out->engine = "p2p"; break;
        case HCCL_ENGINE_NVLS: out->engine = "nvls"; break;
        case HCCL_ENGINE_HOSTCPU: out->engine = "host"; break;
        default: return false;
    }
    out->executor = e.executor;
    out->templ.clear();
    for (auto& t : e.templates) out->templ += t;
    std::transform(out->templ.begin(), out->templ.end(), out->templ.begin(), [](unsigned char c) { return (char)tolower(c); });
    return !out->executor.empty() && !out->templ.empty();
}

// ------------------------------------------------------------------ link model
LinkModel& GlobalLinkModel()
{
    static LinkModel m;
    return m;
}

namespace {
struct UtilPoint { double bytes, util; };
// Utilisation of the per-direction NVLink bandwidth by this library's SM kernels as a function of the bytes one
// rank moves over one peer link in the op.  Values are the measured ratios of the 8-GPU sweep (bench/sweep.py);
// below the first point the curve is latency-bound and extrapolates linearly in size.
const UtilPoint kP2pUtil[] = {{4096, 0.004}, {16384, 0.016}, {65536, 0.06}, {262144, 0.2}, {1048576, 0.45},
                              {4194304, 0.7}, {16777216, 0.84}, {67108864, 0.9}, {268435456, 0.93}};
const UtilPoint kNvlsUtil[] = {{4096, 0.003}, {16384, 0.012}, {65536, 0.05}, {262144, 0.17}, {1048576, 0.42},
                               {4194304, 0.68}, {16777216, 0.8}, {67108864, 0.85}, {268435456, 0.87}};
const UtilPoint kHostUtil[] = {{4096, 0.2}, {65536, 0.6}, {1048576, 0.9}, {16777216, 1.0}};

template <size_t N>
double Interp(const UtilPoint (&t)[N], double bytes)
{
    if (bytes <= t[0].bytes) return std::max(1e-4, t[0].util * bytes / t[0].bytes);
    for (size_t i = 1; i < N; ++i) {
        if (bytes <= t[i].bytes) {
            // interpolate in log(size)
            double f = (std::log(bytes) - std::log(t[i - 1].bytes)) / (std::log(t[i].bytes) - std::log(t[i - 1].bytes));
            return t[i - 1].util + f * (t[i].util - t[i - 1].util);
        }
    }
    return t[N - 1].util;
}
}  // namespace

namespace {
// measured curves per GPU count, loaded from a measurement file; empty = built-in curves
struct LoadedCurves {
    std::map<int, std::vector<UtilPoint>> p2p, nvls;
    std::mutex mu;
};
LoadedCurves& Curves()
{
    static LoadedCurves c;
    return c;
}
double InterpVec(const std::vector<UtilPoint>& t, double bytes)
{
    if (bytes <= t[0].bytes) return std::max(1e-4, t[0].util * bytes / t[0].bytes);
    for (size_t i = 1; i < t.size(); ++i) {
        if (bytes <= t[i].bytes) {
            const double f = (std::log(bytes) - std::log(t[i - 1].bytes)) / (std::log(t[i].bytes) - std::log(t[i - 1].bytes));
            return t[i - 1].util + f * (t[i].util - t[i - 1].util);
        }
    }
    return t.back().util;
}
const std::vector<UtilPoint>* Nearest(const std::map<int, std::vector<UtilPoint>>& m, int nRanks)
{
    const std::vector<UtilPoint>* best = nullptr;
    int bestDist = 1 << 30;
    for (auto& kv : m) {
        const int d = std::abs(kv.first - nRanks);
        if (!kv.second.empty() && d < bestDist) { bestDist = d; best = &kv.second; }
    }
    return best;
}
}  // namespace

double LinkUtilisation(NetType net, double bytes, HcclCommEngine, int nRanks)
{
    if (nRanks > 0 && (net == NetType::MESH_P2P || net == NetType::NVLS_SWITCH)) {
        LoadedCurves& c = Curves();
        std::lock_guard<std::mutex> lk(c.mu);
        const std::vector<UtilPoint>* t = Nearest(net == NetType::MESH_P2P ? c.p2p : c.nvls, nRanks);
        if (t != nullptr) return InterpVec(*t, bytes);
    }
    switch (net) {
        case NetType::MESH_P2P: return Interp(kP2pUtil, bytes);
        case NetType::NVLS_SWITCH: return Interp(kNvlsUtil, bytes);
        case NetType::HOST_MEM: return Interp(kHostUtil, bytes);
        default: return 1.0;
    }
}

bool LoadLinkModelFile(const std::string& path, std::string* err)
{
    std::ifstream f(path);
    if (!f) { if (err) *err = "cannot open " + path; return false; }
    std::stringstream ss;
    ss << f.rdbuf();
    JsonValue root;
    std::string perr;
    const std::string text = ss.str();          // the parser keeps a reference
    JsonParser parser(text);
    if (!parser.Parse(&root, &perr) || root.kind != JsonValue::OBJ) { if (err) *err = "not a JSON object: " + perr; return false; }
    LinkModel lm = GlobalLinkModel();
    if (const JsonValue* link = root.Get("link")) {
        auto num = [&](const char* k, double* out) { const JsonValue* v = link->Get(k); if (v && v->kind == JsonValue::NUM && v->num > 0) *out = v->num; };
        num("p2pGBs", &lm.p2pGBs); num("nvlsGBs", &lm.nvlsGBs); num("nvlsReduceOutGBs", &lm.nvlsReduceOutGBs); num("nvlsStoreGBs", &lm.nvlsStoreGBs);
        num("localCopyGBs", &lm.localCopyGBs); num("localReduceGBs", &lm.localReduceGBs); num("launchUs", &lm.launchUs); num("barrierUs", &lm.barrierUs);
        num("llHopUs", &lm.llHopUs);
    }
    std::map<int, std::vector<UtilPoint>> p2p, nvls;
    if (const JsonValue* u = root.Get("utilisation")) {
        for (const char* kind : {"p2p", "nvls"}) {
            const JsonValue* k = u->Get(kind);
            if (!k || k->kind != JsonValue::OBJ) continue;
            for (auto& kv : k->obj) {
                const int n = atoi(kv.first.c_str());
                if (n < 2 || kv.second.kind != JsonValue::ARR) { if (err) *err = std::string("utilisation.") + kind + ": keys are GPU counts, values arrays of [bytes, utilisation]"; return false; }
                std::vector<UtilPoint> pts;
                for (const JsonValue& pt : kv.second.arr) {
                    if (pt.kind != JsonValue::ARR || pt.arr.size() != 2 || pt.arr[0].num <= 0 || pt.arr[1].num <= 0 || pt.arr[1].num > 1.5 ||
                        (!pts.empty() && pt.arr[0].num <= pts.back().bytes)) {
                        if (err) *err = std::string("utilisation.") + kind + "." + kv.first + ": points must be [bytes, utilisation] with growing bytes and utilisation in (0, 1.5]";
                        return false;
                    }
                    pts.push_back(UtilPoint{pt.arr[0].num, pt.arr[1].num});
                }
                if (!pts.empty()) (std::string(kind) == "p2p" ? p2p : nvls)[n] = pts;
            }
        }
    }
    GlobalLinkModel() = lm;
    LoadedCurves& c = Curves();
    std::lock_guard<std::mutex> lk(c.mu);
    c.p2p = p2p;
    c.nvls = nvls;
    return true;
}

std::string DefaultLinkModelPath()
{
    if (const char* e = getenv("HCCL_LINK_MODEL_FILE")) return e;
    Dl_info info;
    if (dladdr((const void*)&DefaultLinkModelPath, &info) == 0 || info.dli_fname == nullptr) return "";
    std::string lib = info.dli_fname;                       // .../hccl_b200/lib/libhccl_b200.so
    const size_t slash = lib.rfind('/');
    if (slash == std::string::npos) return "";
    const std::string candidate = lib.substr(0, slash) + "/../data/link_model.json";
    std::ifstream f(candidate);
    return f ? candidate : "";
}

double EvalCost(const std::vector<CostCoeff>& segs, CostAgg agg, double bytes, HcclCommEngine engine, int nRanks)
{
    std::map<int, double> groups;
    double floorSum = 0;
    for (const CostCoeff& s : segs) {
        const double util = s.A > 0 ? LinkUtilisation(s.net, bytes * s.ratio, engine, nRanks) : 1.0;
        const double seg = (s.A / util + s.B + s.Bre) * bytes + s.C;
        double& g = groups[s.group];
        g = (agg == CostAgg::MAX) ? std::max(g, seg) : g + seg;
        floorSum += s.D;
    }
    double total = 0;
    for (auto& kv : groups) total += kv.second;
    return std::max(total, floorSum);
}

std::vector<HcclCommEngine> EngineTiers(HcclCommEngine req)
{
    // A requested engine is tried first; the others follow as fallbacks (resource unavailable -> next engine,
    // reference FallbackOp op_common.cc:1343-1351).  In auto mode the two device engines compete by cost in one
    // tier - flagged by HCCL_ENGINE_AUTO as the first element.
    switch (req) {
        case HCCL_ENGINE_P2P: return {HCCL_ENGINE_P2P, HCCL_ENGINE_NVLS, HCCL_ENGINE_HOSTCPU};
        case HCCL_ENGINE_NVLS: return {HCCL_ENGINE_NVLS, HCCL_ENGINE_P2P, HCCL_ENGINE_HOSTCPU};
        case HCCL_ENGINE_HOSTCPU: return {HCCL_ENGINE_HOSTCPU};
        default: return {HCCL_ENGINE_AUTO, HCCL_ENGINE_HOSTCPU};
    }
}

// ------------------------------------------------------------------ tuner host
SelectorState::SelectorState() {}
SelectorState::~SelectorState() { TunerClose(*this); }

void TunerClose(SelectorState& st)
{
    if (st.tunerHandle) dlclose(st.tunerHandle);
    st.tunerHandle = nullptr;
    st.tunerOps = nullptr;
}

static bool HeaderOk(const HcclAbiHeader& h, uint32_t magic, uint32_t version, uint32_t minSize)
{
    // triple check: magic, version not newer than the host, size at least what this host reads
    return h.magicWord == magic && h.version >= 1 && h.version <= version && h.size >= minSize;
}

HcclResult TunerInit(SelectorState& st, const EnvConfig& env, const TopoInfo& topo, const std::string& commName,
                     HcclComm commHandle, uint64_t bufferBytes)
{
    if (st.tunerInitTried) return HCCL_SUCCESS;
    st.tunerInitTried = true;
    if (env.tunerPlugin.empty()) return HCCL_SUCCESS;
    void* h = dlopen(env.tunerPlugin.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) { HCCL_WARNING("tuner plugin '%s' cannot be loaded (%s): selection continues without it", env.tunerPlugin.c_str(), dlerror()); return HCCL_SUCCESS; }
    using GetFn = const HcclTunerPluginOps* (*)();
    GetFn get = (GetFn)dlsym(h, "HcclTunerPluginOpsGet");
    const HcclTunerPluginOps* ops = get ? get() : nullptr;
    if (!ops || !HeaderOk(ops->header, HCCL_TUNER_PLUGIN_OPS_MAGIC_WORD, HCCL_TUNER_PLUGIN_OPS_VERSION, (uint32_t)sizeof(HcclTunerPluginOps)) ||
        !ops->UpdateAlgoCostTable) {
        HCCL_WARNING("tuner plugin '%s' has no valid HcclTunerPluginOpsGet (symbol, ABI header or callbacks): ignored", env.tunerPlugin.c_str());
        dlclose(h);
        return HCCL_SUCCESS;
    }
    HcclTunerTopoInfo ti;
    HcclTunerTopoInfoInit(&ti);
    ti.nRanks = topo.nRanks;
    ti.nNpusPerServer = topo.serverSizes.empty() ? topo.nRanks : topo.serverSizes[0];
    ti.nServers = topo.nServers;
    ti.nPods = topo.nPods;
    ti.nSuperPods = topo.nPods;
    HcclTunerCommInfo ci;
    HcclTunerCommInfoInit(&ci);
    ci.commName = commName.c_str();
    ci.bufferSize = bufferBytes;
    if (ops->Create) {
        void* ctx = nullptr;
        uint32_t ctxSize = 0;
        HcclResult r = ops->Create(commHandle, &ci, &ti, &ctx, &ctxSize);
        if (r != HCCL_SUCCESS) {
            HCCL_WARNING("tuner plugin Create failed (%s): plugin disabled for comm %s", ResultString(r), commName.c_str());
            if (ctx) free(ctx);
            dlclose(h);
            return HCCL_SUCCESS;
        }
        if (ctx && ctxSize) st.tunerCtx.assign((uint8_t*)ctx, (uint8_t*)ctx + ctxSize);  // host-owned copy
        if (ctx) free(ctx);
    }
    st.tunerHandle = h;
    st.tunerOps = ops;
    HCCL_INFO("tuner plugin '%s' active for comm %s", env.tunerPlugin.c_str(), commName.c_str());
    return HCCL_SUCCESS;
}

// ------------------------------------------------------------------ model + table
namespace {

bool EngineAvailable(const AlgEntry& a, const TopoInfo& topo, std::string* why)
{
    if (a.engine == HCCL_ENGINE_NVLS && !topo.nvls) { *why = "engine: NVLS multicast not available on this communicator"; return false; }
    if ((a.engine == HCCL_ENGINE_P2P || a.engine == HCCL_ENGINE_NVLS) && topo.level0Link == LinkKind::HOST_MEM && topo.deviceName.empty()) {
        *why = "engine: no GPU behind this communicator";
        return false;
    }
    if (a.engine == HCCL_ENGINE_HOSTCPU && !(topo.level0Link == LinkKind::HOST_MEM && topo.deviceName.empty())) {
        *why = "engine: host engine only drives host-memory communicators";
        return false;
    }
    return true;
}

bool TopoMatches(const AlgEntry& a, const TopoInfo& topo, std::string* why)
{
    const AlgAttrs& t = a.attrs;
    const uint32_t levels = topo.nPods > 1 ? 3 : (topo.nServers > 1 ? 2 : 1);
    // an algorithm with fewer levels than the topology treats the extra levels as one flat group, which is legal;
    // more levels than the topology has is not
    // Servers of different sizes have no level-1 groups of equal local index: the hierarchical forms are out and the
    // flat forms run across the levels as one group (the reference falls back to a flat NHR when the server sizes
    // share no common divisor, topo_host.cc:662-684).
    if (t.enforceMaxLevels && levels > t.maxLevels && topo.symmetric) { *why = "topo: flat algorithm on a " + std::to_string(levels) + "-level topology"; return false; }
    if (t.minLevels > levels) { *why = "topo: needs " + std::to_string(t.minLevels) + " levels, topology has " + std::to_string(levels); return false; }
    if (!(t.level0Shapes & (1u << (int)topo.level0))) { *why = "topo: level-0 shape not supported"; return false; }
    if (t.maxRankSize && topo.nRanks > t.maxRankSize) { *why = "topo: more than " + std::to_string(t.maxRankSize) + " ranks"; return false; }
    if (topo.nRanks < t.minRankSize) { *why = "topo: fewer than " + std::to_string(t.minRankSize) + " ranks"; return false; }
    if (t.powerOfTwoRanksOnly && (topo.nRanks & (topo.nRanks - 1))) { *why = "topo: rank count is not a power of two"; return false; }
    if (t.minLevels > 1 && !topo.symmetric) { *why = "topo: hierarchical algorithm needs symmetric servers"; return false; }
    if (t.topoCustomCheck && !t.topoCustomCheck(topo, why)) return false;
    return true;
}

void BuildModel(SelectorState& st, const TopoInfo& topo)
{
    EnsureAlgorithmsRegistered();
    // link parameters and utilisation curves measured on the box, when a measurement file is there (once per process)
    static std::once_flag linkModelOnce;
    std::call_once(linkModelOnce, [] {
        const std::string path = DefaultLinkModelPath();
        if (path.empty()) return;
        std::string err;
        if (LoadLinkModelFile(path, &err)) HCCL_CONFIG_INFO(LOG_MOD_ALG, "link model loaded from %s", path.c_str());
        else HCCL_WARNING("link model file %s ignored: %s", path.c_str(), err.c_str());
    });
    const auto& all = AlgRegistry::Instance().All();
    st.modelDropReason.assign(all.size(), "");
    for (auto& v : st.modelAlgs) v.clear();
    for (size_t i = 0; i < all.size(); ++i) {
        std::string why;
        if (!EngineAvailable(all[i], topo, &why) || !TopoMatches(all[i], topo, &why)) { st.modelDropReason[i] = why; continue; }
        st.modelAlgs[all[i].op].push_back((int)i);
    }
    st.modelReady = true;
}

bool OpMatches(const AlgEntry& a, const OpDesc& op, const TopoInfo& topo, std::string* why)
{
    const AlgAttrs& t = a.attrs;
    const bool reduces = op.op == HCCL_CMD_ALLREDUCE || op.op == HCCL_CMD_REDUCE || op.op == HCCL_CMD_REDUCE_SCATTER ||
                         op.op == HCCL_CMD_REDUCE_SCATTER_V;
    if (op.dtype != HCCL_DATA_TYPE_RESERVED && (int)op.dtype < 64 && !(t.dtypeMask & (1ull << (int)op.dtype))) { *why = "op: data type not supported"; return false; }
    if (reduces) {
        if (op.redOp == HCCL_REDUCE_PROD && !t.supportProd) { *why = "op: PROD not supported"; return false; }
        if ((op.redOp == HCCL_REDUCE_MAX || op.redOp == HCCL_REDUCE_MIN) && !t.supportMaxMin) { *why = "op: MAX/MIN not supported"; return false; }
        // The order of a reduction only shows in the result for floating-point SUM / PROD over more than two ranks
        // (reference IsNeedStrictModeForOrderPreserved, order_preserved_common.h:104-114): integer and MAX / MIN
        // reductions are exact in any order, and two values have one order.
        const bool isFloat = op.dtype == HCCL_DATA_TYPE_FP16 || op.dtype == HCCL_DATA_TYPE_BFP16 || op.dtype == HCCL_DATA_TYPE_FP32 ||
                             op.dtype == HCCL_DATA_TYPE_FP64 || op.dtype == HCCL_DATA_TYPE_FP8E4M3 || op.dtype == HCCL_DATA_TYPE_FP8E5M2 ||
                             op.dtype == HCCL_DATA_TYPE_HIF8;
        const bool orderShows = isFloat && (op.redOp == HCCL_REDUCE_SUM || op.redOp == HCCL_REDUCE_PROD) && op.nRanks > 2;
        if (op.det == Deterministic::STRICT && orderShows && !t.orderPreserved) { *why = "op: reduction order not fixed (HCCL_DETERMINISTIC=strict)"; return false; }
        if (op.det == Deterministic::ON && !t.deterministic) { *why = "op: not run-to-run deterministic"; return false; }
    }
    if (op.inPlace && !t.supportInplace) { *why = "op: in-place not supported"; return false; }
    if (op.bytes < t.minBytes || op.bytes > t.maxBytes) { *why = "op: message size outside [" + std::to_string(t.minBytes) + ", " + std::to_string(t.maxBytes) + "]"; return false; }
    if (t.needsAligned16 && !op.aligned16) { *why = "op: buffers are not 16-byte aligned"; return false; }
    if (t.needsRegisteredOut && !op.outRegistered) { *why = "op: output is not symmetric memory"; return false; }
    if (op.isMc2 && !t.supportMc2) { *why = "op: not usable from fused matmul kernels"; return false; }
    if (op.castScale != t.castScale) { *why = t.castScale ? "op: a cast + scale form, the call asks for neither" : "op: the call casts or scales"; return false; }
    if (t.opCustomCheck && !t.opCustomCheck(op, topo, why)) return false;
    return true;
}

bool MatchesPreference(const AlgEntry& a, const AlgoLevelConfig& pref)
{
    if (!pref.specified) return false;
    // level1 names the algorithm across level-0 groups; on a single box there is only level 0 and a level1 entry
    // applies to the flat group, which is how the reference treats NHR / ring / H-D_R for a one-level topology.
    for (int l = 0; l < kAlgoLevels; ++l) {
        AlgoType want = pref.level[l];
        if (want == AlgoType::DEFAULT || want == AlgoType::NA) continue;
        if (want == a.family) return true;
    }
    return false;
}

}  // namespace

std::string FormatCostTable(const Selection& s)
{
    std::ostringstream os;
    const auto& all = AlgRegistry::Instance().All();
    for (const CostRow& r : s.table) {
        os << "  " << all[(size_t)r.algIndex].name << ": ";
        if (r.viable) os << r.cost << " us" << (r.byThreshold ? " [threshold]" : r.preferred ? " [HCCL_ALGO]" : "") << (r.tunerTouched ? " [tuner]" : "");
        else os << "filtered (" << r.reason << ")";
        if (r.algIndex == s.algIndex) os << "  <= selected";
        os << "\n";
    }
    return os.str();
}

HcclResult SelectAlgorithm(SelectorState& st, const TopoInfo& topo, const EnvConfig& env, const OpDesc& op,
                           const std::string& commName, HcclComm commHandle, uint64_t bufferBytes, Selection* out)
{
    if (!st.modelReady) BuildModel(st, topo);
    TunerInit(st, env, topo, commName, commHandle, bufferBytes);
    const auto& all = AlgRegistry::Instance().All();
    out->table.clear();
    out->algIndex = -1;
    out->alg = nullptr;
    if (op.op <= HCCL_CMD_INVALID || op.op >= HCCL_CMD_MAX) return HCCL_E_PARA;
    // Phase 1: op filter + cost
    for (int idx : st.modelAlgs[op.op]) {
        CostRow row;
        row.algIndex = idx;
        std::string why;
        if (!OpMatches(all[(size_t)idx], op, topo, &why)) { row.reason = why; out->table.push_back(row); continue; }
        row.viable = true;
        row.cost = all[(size_t)idx].costCoeff ? EvalCost(all[(size_t)idx].costCoeff(topo, op), all[(size_t)idx].agg, (double)op.bytes, all[(size_t)idx].engine, (int)topo.nRanks) : 1e9;
        out->table.push_back(row);
    }
    // Phase 2: HCCL_ALGO is a preference, not a hard filter: if any viable algorithm matches, only those compete
    const AlgoLevelConfig& pref = env.algo.For(op.op);
    bool anyPref = false;
    for (CostRow& r : out->table)
        if (r.viable && MatchesPreference(all[(size_t)r.algIndex], pref)) { r.preferred = true; anyPref = true; }
    // Phase 2b: the threshold tree names one algorithm (HCCL_SELECTOR_MODE=threshold, and always for calls made on
    // behalf of fused matmul kernels, as the reference does for MC2, op_common.cc:225-230).  HCCL_ALGO still wins.
    if (!anyPref && (env.thresholdSelector || op.isMc2)) {
        const std::string name = ThresholdSelect(ThresholdInputOf(topo, op));
        for (CostRow& r : out->table)
            if (r.viable && all[(size_t)r.algIndex].name == name) { r.preferred = r.byThreshold = true; anyPref = true; }
        if (!name.empty() && !anyPref)
            HCCL_INFO("threshold tree names %s, which cannot run this call: cost model decides", name.c_str());
    }
    if (pref.specified && !anyPref)
        HCCL_WARNING("HCCL_ALGO names no algorithm that can run this %d-rank op (%llu bytes): automatic selection", op.nRanks, (unsigned long long)op.bytes);
    // Phase 3: tuner
    if (st.tunerOps && !st.tunerDisabled) {
        std::vector<HcclTunerAlgoCostEntry> entries;
        std::vector<AlgNameDims> dims(out->table.size());
        std::vector<size_t> rowOf;
        for (size_t i = 0; i < out->table.size(); ++i) {
            if (!out->table[i].viable) continue;
            const AlgEntry& a = all[(size_t)out->table[i].algIndex];
            if (!MapAlgName(a, &dims[i])) continue;
            HcclTunerAlgoCostEntry e;
            HcclTunerAlgoCostEntryInit(&e);
            e.algName = a.name.c_str();
            e.engineName = dims[i].engine.c_str();
            e.executorName = dims[i].executor.c_str();
            e.templateName = dims[i].templ.c_str();
            e.cost = (float)out->table[i].cost;
            entries.push_back(e);
            rowOf.push_back(i);
        }
        if (!entries.empty()) {
            HcclTunerCollOpInfo oi;
            HcclTunerCollOpInfoInit(&oi);
            oi.nBytes = op.bytes; oi.collType = op.op; oi.dataType = op.dtype; oi.reduceOp = op.redOp;
            std::vector<HcclTunerAlgoCostEntry> before = entries;
            bool matched = false;
            auto t0 = std::chrono::steady_clock::now();
            HcclResult r = st.tunerOps->UpdateAlgoCostTable(st.tunerCtx.empty() ? nullptr : st.tunerCtx.data(), &oi, entries.data(), (uint32_t)entries.size(), &matched);
            double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            // a tuner that repeatedly takes > 100 ms per call is switched off after 3 such calls (tuner_setup.h:28-46)
            if (ms > 100.0 && ++st.tunerSlowCalls >= 3) { st.tunerDisabled = true; HCCL_WARNING("tuner plugin disabled: 3 calls slower than 100 ms"); }
            if (r == HCCL_SUCCESS && matched) {
                for (size_t k = 0; k < entries.size(); ++k) {
                    if (entries[k].cost == before[k].cost) continue;
                    CostRow& row = out->table[rowOf[k]];
                    row.tunerTouched = true;
                    row.cost = entries[k].cost;
                    if (entries[k].cost < 0) { row.viable = false; row.reason = "tuner: disabled"; }
                }
            } else if (r != HCCL_SUCCESS) {
                HCCL_WARNING("tuner plugin UpdateAlgoCostTable failed (%s): model costs kept", ResultString(r));
            }
        }
    }
    // Phase 4: best engine tier, min cost, ties -> deeper form, then first registered
    const std::vector<HcclCommEngine> tiers = EngineTiers(op.engine);
    for (HcclCommEngine tier : tiers) {
        int best = -1;
        bool tie = false;
        for (size_t i = 0; i < out->table.size(); ++i) {
            const CostRow& r = out->table[i];
            if (!r.viable) continue;
            const AlgEntry& a = all[(size_t)r.algIndex];
            const bool inTier = (tier == HCCL_ENGINE_AUTO) ? (a.engine == HCCL_ENGINE_P2P || a.engine == HCCL_ENGINE_NVLS) : a.engine == tier;
            if (!inTier) continue;
            if (anyPref && !r.preferred) continue;
            if (best < 0 || r.cost < out->table[(size_t)best].cost) { best = (int)i; tie = false; }
            else if (r.cost == out->table[(size_t)best].cost) {
                // equal cost: the form written for more topology levels is the more specific one and wins quietly;
                // between forms of the same depth the first registered one stays (and the tie is reported)
                const uint32_t depth = a.attrs.minLevels, bestDepth = all[(size_t)out->table[(size_t)best].algIndex].attrs.minLevels;
                if (depth > bestDepth) { best = (int)i; tie = false; }
                else if (depth == bestDepth) tie = true;
            }
        }
        if (best >= 0) {
            // once per operator and communicator, and at most a handful per process: threads-as-ranks share the finding
            static std::atomic<uint32_t> processWide[HCCL_CMD_MAX];
            if (tie && !st.tieWarned[op.op] && (st.tieWarned[op.op] = true) && processWide[op.op].fetch_add(1) < 2) {
                HCCL_WARNING("cost tie for op %d at %llu bytes: first registered algorithm wins (said once per operator)", (int)op.op, (unsigned long long)op.bytes);
            }
            out->algIndex = out->table[(size_t)best].algIndex;
            out->alg = &all[(size_t)out->algIndex];
            out->costUs = out->table[(size_t)best].cost;
            ++st.selections;
            HCCL_CONFIG_INFO(LOG_MOD_ALG, "comm %s op %d bytes %llu ranks %u -> %s (%.2f us)\n%s", commName.c_str(), (int)op.op,
                             (unsigned long long)op.bytes, op.nRanks, out->alg->name.c_str(), out->costUs, FormatCostTable(*out).c_str());
            return HCCL_SUCCESS;
        }
    }
    // nothing survived: say which filter removed each algorithm
    std::ostringstream os;
    for (const CostRow& r : out->table) os << "\n  " << all[(size_t)r.algIndex].name << ": " << r.reason;
    for (size_t i = 0; i < all.size(); ++i)
        if (all[i].op == op.op && !st.modelDropReason[i].empty()) os << "\n  " << all[i].name << ": " << st.modelDropReason[i];
    HCCL_ERROR("no algorithm can run op %d (%llu bytes, dtype %d, %u ranks):%s", (int)op.op, (unsigned long long)op.bytes, (int)op.dtype, op.nRanks, os.str().c_str());
    return HCCL_E_NOT_SUPPORT;
}

}  // namespace hccl
