// Host-engine communicators: creation, operator execution (selection + sole
// executor loop + template run) and registration of the host algorithms.
#include "host_comm.h"
#include <algorithm>
#include <chrono>
#include <cstring>
#include <map>
#include <sstream>
#include <thread>
#include "../core/comm.h"
#include "../core/json.h"
#include "../core/log.h"
#include "../core/plan_cache.h"
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "../select/selector.h"
#include "hccl/hccl_ext.h"
#include "host_tree.h"
#include "host_world.h"

namespace hccl {

namespace {

bool ParseTopoMeta(const char* json, uint32_t nRanks, TopoMeta* out, std::string* err)
{
    out->clear();
    if (!json || !*json) {
        std::vector<uint32_t> dev(nRanks);
        for (uint32_t i = 0; i < nRanks; ++i) dev[i] = i;
        out->push_back({dev});
        return true;
    }
    JsonValue v;
    if (!JsonParser(json).Parse(&v, err)) return false;
    if (v.kind != JsonValue::ARR) { *err = "topology literal must be an array of pods"; return false; }
    uint32_t total = 0;
    for (auto& pod : v.arr) {
        if (pod.kind != JsonValue::ARR) { *err = "a pod must be an array of servers"; return false; }
        std::vector<std::vector<uint32_t>> servers;
        for (auto& srv : pod.arr) {
            if (srv.kind != JsonValue::ARR) { *err = "a server must be an array of device ids"; return false; }
            std::vector<uint32_t> devs;
            for (auto& d : srv.arr) { unsigned long long x; if (!d.AsU64(&x)) { *err = "device ids must be numbers"; return false; } devs.push_back((uint32_t)x); ++total; }
            servers.push_back(devs);
        }
        out->push_back(servers);
    }
    if (total != nRanks) { *err = "topology literal lists " + std::to_string(total) + " devices for " + std::to_string(nRanks) + " ranks"; return false; }
    return true;
}

uint64_t InBytes(const OpParam& p, uint32_t n)
{
    const uint64_t es = DataTypeSize(p.dtype);
    switch (p.op) {
        case HCCL_CMD_REDUCE_SCATTER: case HCCL_CMD_SCATTER: return p.count * es * n;
        case HCCL_CMD_REDUCE_SCATTER_V: { uint64_t m = 0; for (uint32_t q = 0; q < n; ++q) m = std::max(m, (p.sdispls[q] + p.sendCounts[q]) * es); return m; }
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: { uint64_t m = 0; for (uint32_t q = 0; q < n; ++q) m = std::max(m, (p.sdispls[q] + p.sendCounts[q]) * es); return m; }
        case HCCL_CMD_BARRIER: case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: case HCCL_CMD_BATCH_SEND_RECV: return 0;
        default: return p.count * es;
    }
}
uint64_t OutBytes(const OpParam& p, uint32_t n)
{
    const uint64_t es = DataTypeSize(p.dtype), res = DataTypeSize(p.recvType);
    switch (p.op) {
        case HCCL_CMD_ALLGATHER: return p.count * es * n;
        case HCCL_CMD_ALLGATHER_V: { uint64_t m = 0; for (uint32_t q = 0; q < n; ++q) m = std::max(m, (p.rdispls[q] + p.recvCounts[q]) * es); return m; }
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: { uint64_t m = 0; for (uint32_t q = 0; q < n; ++q) m = std::max(m, (p.rdispls[q] + p.recvCounts[q]) * res); return m; }
        case HCCL_CMD_BARRIER: case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: case HCCL_CMD_BATCH_SEND_RECV: return 0;
        default: return p.count * es;
    }
}

HostOpDesc Desc(const OpParam& p)
{
    HostOpDesc d;
    d.op = p.op; d.dtype = p.dtype; d.redOp = p.redOp; d.count = p.count; d.root = p.root;
    d.sendCounts = p.sendCounts; d.sdispls = p.sdispls; d.recvCounts = p.recvCounts; d.rdispls = p.rdispls;
    return d;
}

}  // namespace

HcclResult HostWorldCreate(uint32_t nRanks, const char* topoJson, const HcclCommConfig* cfg, CommImpl** comms)
{
    if (nRanks == 0 || nRanks > 4096) return HCCL_E_PARA;
    TopoMeta meta;
    std::string err;
    if (!ParseTopoMeta(topoJson, nRanks, &meta, &err)) { HCCL_ERROR("host communicator: %s", err.c_str()); return HCCL_E_PARA; }
    EffectiveConfig eff;
    CHK_RET(MergeConfig(GetEnvConfig(), cfg, &eff));
    // the per-rank scratch is host memory: default 64 MiB unless configured
    const bool sized = (cfg && cfg->hcclBufferSize) || GetEnvConfig().bufferSizeMiB;
    const uint64_t scratch = sized ? eff.bufferBytes : (64ull << 20);
    auto world = std::make_shared<HostWorld>(nRanks, meta, scratch, eff.execTimeoutNs);
    for (uint32_t r = 0; r < nRanks; ++r) {
        CommImpl* c = new CommImpl();
        c->rank = (int)r;
        c->nRanks = (int)nRanks;
        c->device = -1;
        c->cfg = eff;
        char nm[64];
        snprintf(nm, sizeof(nm), "hccl_host_%p", (void*)world.get());
        c->name = eff.commName.empty() ? nm : eff.commName;
        GroupRegister(c);
        c->hostComm = new HostRank(world, r);
        c->topo.reset(new TopoInfo(world->Topo(r)));
        c->selector.reset(new SelectorState());
        c->plans.reset(new PlanCache());
        comms[r] = c;
    }
    return HCCL_SUCCESS;
}

void HostRankRelease(HostRank* r) { delete r; }

HcclResult HostExecOp(CommImpl* c, OpParam& p)
{
    HostWorld& w = *c->hostComm->world;
    const uint32_t rank = c->hostComm->rank, n = w.nRanks();
    // selection (identical on every rank: same inputs)
    OpDesc d;
    d.op = p.op; d.dtype = p.dtype; d.redOp = p.redOp; d.root = p.root; d.nRanks = n;
    d.det = c->cfg.deterministic;
    d.engine = HCCL_ENGINE_HOSTCPU;
    d.bytes = std::max(InBytes(p, n), OutBytes(p, n));
    d.inPlace = p.send == p.recv;
    Selection sel;
    CHK_RET(SelectAlgorithm(*c->selector, *c->topo, GetEnvConfig(), d, c->name, (HcclComm)c, w.scratchBytes(), &sel));
    p.algName = sel.alg->name;
    const int alg = sel.alg->hostAlg;
    const uint64_t es = DataTypeSize(p.dtype);

    // sole-executor loop for the contiguous operators: bytes per loop = floor(scratch / multiple / 128) * 128
    const bool chunkable = p.op == HCCL_CMD_ALLREDUCE || p.op == HCCL_CMD_BROADCAST || p.op == HCCL_CMD_REDUCE;
    uint64_t perLoop = p.count;
    if (chunkable && es) {
        const uint64_t mult = HostScratchMultiple(alg, n) * 2;    // templates that keep W in scratch use half of it
        const uint64_t maxBytes = w.scratchBytes() / mult / 128 * 128;
        if (maxBytes == 0) return HCCL_E_MEMORY;
        perLoop = std::min<uint64_t>(p.count, std::max<uint64_t>(1, maxBytes / es));
    } else if (d.bytes * 2 > w.scratchBytes() && p.op != HCCL_CMD_BARRIER && p.op != HCCL_CMD_SEND && p.op != HCCL_CMD_RECEIVE &&
               p.op != HCCL_CMD_BATCH_SEND_RECV && p.op != HCCL_CMD_ALLGATHER && p.op != HCCL_CMD_ALLGATHER_V && p.op != HCCL_CMD_ALLTOALL &&
               p.op != HCCL_CMD_ALLTOALLV && p.op != HCCL_CMD_ALLTOALLVC && p.op != HCCL_CMD_SCATTER) {
        HCCL_ERROR("host engine: %s of %llu bytes needs more than the %llu-byte scratch buffer (raise HCCL_BUFFSIZE)", CmdName(p.op),
                   (unsigned long long)d.bytes, (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    HcclResult result = HCCL_SUCCESS;
    for (uint64_t off = 0; off < std::max<uint64_t>(p.count, 1); off += std::max<uint64_t>(perLoop, 1)) {
        OpParam sub = p;
        if (chunkable) {
            sub.count = std::min(perLoop, p.count - off);
            sub.send = (const char*)p.send + off * es;
            sub.recv = p.recv ? (char*)p.recv + off * es : nullptr;
        }
        HostOpDesc hd = Desc(sub);
        const void* in = sub.send;
        void* out = sub.recv;
        if (p.op == HCCL_CMD_BROADCAST) { in = sub.recv; }
        // Operator retry (HCCL_OP_RETRY_ENABLE, HCCL_OP_RETRY_PARAMS; reference HCCL_OP_RETRY_ENABLE.md:7-42): an
        // attempt that ended in a timeout or a peer's failure is issued again from its input after every rank has
        // reached the recovery point.  The input must still be intact, so in-place calls are not retried.
        const EnvConfig& env = GetEnvConfig();
        const bool inputKept = p.op != HCCL_CMD_BROADCAST && sub.send != sub.recv;
        HcclResult r = HCCL_SUCCESS;
        for (uint32_t attempt = 0;; ++attempt) {
            r = w.Enter(rank, hd, in, out, InBytes(sub, n), OutBytes(sub, n));
            if (r == HCCL_SUCCESS) r = RunHostAlgorithm(w, rank, alg, sub);
            HcclResult l = w.Leave(rank);
            if (r == HCCL_SUCCESS) r = l;
            if (r == HCCL_SUCCESS || !(r == HCCL_E_TIMEOUT || r == HCCL_E_REMOTE) || !(env.retryL1 || env.retryL2) || !inputKept) break;
            if (attempt >= env.retryMaxCnt) { r = HCCL_E_OPRETRY_FAIL; break; }
            HCCL_WARNING("host rank %u: %s failed (%s), retry %u of %u", rank, CmdName(p.op), ResultString(r), attempt + 1, env.retryMaxCnt);
            const uint32_t pauseMs = attempt == 0 ? env.retryHoldMs : env.retryIntervalMs;
            if (pauseMs) std::this_thread::sleep_for(std::chrono::milliseconds(pauseMs));
            if (w.Recover(rank) != HCCL_SUCCESS) { r = HCCL_E_OPRETRY_FAIL; break; }
        }
        if (r != HCCL_SUCCESS) { result = r; break; }
        if (!chunkable) break;
    }
    if (result != HCCL_SUCCESS) c->status_.store(HCCL_COMM_STATUS_ERROR);
    return result;
}

// ------------------------------------------------------------------ registration
namespace {

constexpr uint64_t Bit(HcclDataType t) { return 1ull << (int)t; }
constexpr uint64_t kReduceTypes = Bit(HCCL_DATA_TYPE_INT8) | Bit(HCCL_DATA_TYPE_INT16) | Bit(HCCL_DATA_TYPE_INT32) | Bit(HCCL_DATA_TYPE_INT64) |
                                  Bit(HCCL_DATA_TYPE_UINT64) | Bit(HCCL_DATA_TYPE_FP16) | Bit(HCCL_DATA_TYPE_BFP16) | Bit(HCCL_DATA_TYPE_FP32) |
                                  Bit(HCCL_DATA_TYPE_FP64);

struct HostAlgSpec {
    const char* name;
    HcclCMDType op;
    int hostAlg;
    const char* executor;
    std::vector<std::string> templates;
    AlgoType family;
    uint32_t minLevels;
    bool reduces;
    // cost shape: steps (latency terms) and the fraction of the message that crosses a link per rank
    std::function<double(double p)> steps, traffic;
    bool orderPreserved;
};

double Log2Ceil(double p) { return (double)CeilLog2((uint32_t)p); }

void Reg(const HostAlgSpec& s)
{
    AlgEntry e;
    e.name = s.name;
    e.op = s.op;
    e.engine = HCCL_ENGINE_HOSTCPU;
    e.executor = s.executor;
    e.templates = s.templates;
    e.hostAlg = s.hostAlg;
    e.family = s.family;
    e.attrs.minLevels = s.minLevels;
    e.attrs.maxLevels = 3;
    // operators with hierarchical forms: their flat forms stay on one-level topologies
    if (s.minLevels == 1 && std::string(s.executor) != "orderpreserved" && std::string(s.executor) != "tree" &&
        (s.op == HCCL_CMD_ALLREDUCE || s.op == HCCL_CMD_REDUCE_SCATTER || s.op == HCCL_CMD_ALLGATHER || s.op == HCCL_CMD_BROADCAST || s.op == HCCL_CMD_REDUCE)) {
        e.attrs.maxLevels = 1;
        e.attrs.enforceMaxLevels = true;
    }
    if (s.reduces) e.attrs.dtypeMask = kReduceTypes;
    e.attrs.orderPreserved = s.orderPreserved;
    auto steps = s.steps, traffic = s.traffic;
    e.costCoeff = [steps, traffic](const TopoInfo& t, const OpDesc&) {
        const LinkModel& lm = GlobalLinkModel();
        const double p = (double)t.nRanks;
        CostCoeff c;
        c.A = traffic(p) / (lm.hostMemGBs * 1e3);
        c.C = steps(p) * lm.hostStepUs;
        c.net = NetType::HOST_MEM;
        c.ratio = 1.0 / p;
        return std::vector<CostCoeff>{c};
    };
    if (std::string(s.executor) == "concurrent") {
        // Two link sets side by side: the slower part decides (CostAggMode::MAX, executor_v2_base.h:130-141).  Host
        // memory is ONE link class, so the two parts share it and their times add up; MAX is for a topology whose
        // parts really run on separate links.
        e.agg = CostAgg::SUM;
        e.costCoeff = [steps, traffic](const TopoInfo& t, const OpDesc&) {
            const LinkModel& lm = GlobalLinkModel();
            const double p = (double)t.nRanks;
            CostCoeff a, b;
            a.A = traffic(p) / 3.0 / (lm.hostMemGBs * 1e3);           // mesh part: 56 / (56 + 112) of the data, three steps
            a.C = 3.0 * lm.hostStepUs;
            b.A = traffic(p) * 2.0 / 3.0 / (lm.hostMemGBs * 1e3);     // NHR part
            b.C = (steps(p) + 1.0) * lm.hostStepUs;                    // + the fork / join of the second queue
            a.net = b.net = NetType::HOST_MEM;
            a.ratio = b.ratio = 1.0 / p;
            return std::vector<CostCoeff>{a, b};
        };
    }
    if (std::string(s.executor) == "tree") {
        e.attrs.opCustomCheck = [](const OpDesc&, const TopoInfo&, std::string* why) {
            std::unique_ptr<AlgoTreeNode> tree;
            std::string err;
            const std::string& text = GetEnvConfig().algoTree;
            if (text.empty()) { *why = "op: HCCL_ALGO_TREE is not set"; return false; }
            if (!ParseAlgoTree(text, &tree, &err)) { *why = "op: HCCL_ALGO_TREE: " + err; return false; }
            return true;
        };
    }
    AlgRegistry::Instance().Register(std::move(e));
}

}  // namespace

void RegisterHostAlgorithms()
{
    auto P1 = [](double p) { return p - 1; };
    auto TwoP1 = [](double p) { return 2 * (p - 1); };
    auto L = [](double p) { return Log2Ceil(p); };
    auto TwoL = [](double p) { return 2 * Log2Ceil(p); };
    auto Two = [](double) { return 2.0; };
    auto Three = [](double) { return 3.0; };
    auto rs = [](double p) { return (p - 1) / p; };
    auto ar = [](double p) { return 2 * (p - 1) / p; };
    auto full = [](double p) { return p - 1; };
    auto one = [](double) { return 1.0; };
    // AllReduce
    // Last field: the order in which an element's contributions are folded is fixed and does not depend on the message
    // size or on the element's position (HCCL_DETERMINISTIC=strict admits only those).  Every host algorithm is
    // run-to-run deterministic; ring / NHR / RHD / two-shot / hierarchical forms fold in an order that depends on the
    // slice an element falls into.
    Reg({"HostAllReduceSoleMeshOneShot", HCCL_CMD_ALLREDUCE, HALG_AR_MESH_ONESHOT, "sole", {"MeshOneShot"}, AlgoType::ONESHOT, 1, true, Two, full, true});
    Reg({"HostAllReduceSoleMeshTwoShot", HCCL_CMD_ALLREDUCE, HALG_AR_MESH_TWOSHOT, "sole", {"MeshTwoShot"}, AlgoType::MESH, 1, true, Three, ar, false});
    Reg({"HostAllReduceSoleRing", HCCL_CMD_ALLREDUCE, HALG_AR_RING, "sole", {"Ring"}, AlgoType::RING, 1, true, TwoP1, ar, false});
    Reg({"HostAllReduceSoleRHD", HCCL_CMD_ALLREDUCE, HALG_AR_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, true, TwoL, ar, false});
    Reg({"HostAllReduceSoleNHR", HCCL_CMD_ALLREDUCE, HALG_AR_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, true, TwoL, ar, false});
    Reg({"HostAllReduceStrictOrderedMesh", HCCL_CMD_ALLREDUCE, HALG_AR_ORDER_PRESERVED, "orderpreserved", {"OrderPreservedGroup"}, AlgoType::AHC, 1, true, Three, full, true});
    // three levels first: on a topology with pods it wins the tie with the two-level forms, elsewhere it is filtered
    Reg({"HostAllReduceSequenceMeshNHRNHR", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ3_MESH_NHR_NHR, "sequence", {"Mesh", "NHR", "NHR"}, AlgoType::NHR, 3, true, TwoL, ar, false});
    Reg({"HostAllReduceSequenceMeshRing", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ_MESH_RING, "sequence", {"Mesh", "Ring"}, AlgoType::RING, 2, true, TwoP1, ar, false});
    Reg({"HostAllReduceSequenceMeshNHR", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ_MESH_NHR, "sequence", {"Mesh", "NHR"}, AlgoType::NHR, 2, true, TwoL, ar, false});
    Reg({"HostAllReduceSequenceMeshRHD", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ_MESH_RHD, "sequence", {"Mesh", "RHD"}, AlgoType::HD_R, 2, true, TwoL, ar, false});
    // one physical level folded into a grid (squeeze 2-D match): flat topologies only; one step more than the plain
    // two-shot so that automatic selection keeps that one
    Reg({"HostAllReduceSequenceSqueeze2DMeshMesh", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ_SQUEEZE2D_MESH_MESH, "sequence", {"Mesh", "Mesh"}, AlgoType::HIER, 1, true,
         [](double) { return 4.0; }, ar, false});
    Reg({"HostAllReduceParallelMeshNHR", HCCL_CMD_ALLREDUCE, HALG_AR_PARALLEL_MESH_NHR, "parallel", {"Mesh", "NHR"}, AlgoType::PIPELINE, 2, true, TwoL, ar, false});
    // ReduceScatter (+V)
    Reg({"HostReduceScatterSoleMesh", HCCL_CMD_REDUCE_SCATTER, HALG_RS_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, true, Two, rs, false});
    Reg({"HostReduceScatterSoleRing", HCCL_CMD_REDUCE_SCATTER, HALG_RS_RING, "sole", {"Ring"}, AlgoType::RING, 1, true, P1, rs, false});
    Reg({"HostReduceScatterSoleRHD", HCCL_CMD_REDUCE_SCATTER, HALG_RS_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, true, L, rs, false});
    Reg({"HostReduceScatterSoleNHR", HCCL_CMD_REDUCE_SCATTER, HALG_RS_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, true, L, rs, false});
    Reg({"HostReduceScatterStrictOrderedMesh", HCCL_CMD_REDUCE_SCATTER, HALG_RS_ORDER_PRESERVED, "orderpreserved", {"OrderPreservedGroup"}, AlgoType::AHC, 1, true, Three, full, true});
    // three levels first: on a topology with pods it wins the tie with the two-level form, elsewhere it is filtered
    Reg({"HostReduceScatterSequenceMeshNHRNHR", HCCL_CMD_REDUCE_SCATTER, HALG_RS_SEQ3_MESH_NHR_NHR, "sequence", {"NHR", "NHR", "Mesh"}, AlgoType::NHR, 3, true, L, rs, false});
    Reg({"HostReduceScatterSequenceMeshNHR", HCCL_CMD_REDUCE_SCATTER, HALG_RS_SEQ_MESH_NHR, "sequence", {"NHR", "Mesh"}, AlgoType::NHR, 2, true, L, rs, false});
    Reg({"HostReduceScatterSequenceMeshRing", HCCL_CMD_REDUCE_SCATTER, HALG_RS_SEQ_MESH_RING, "sequence", {"Ring", "Mesh"}, AlgoType::RING, 2, true, P1, rs, false});
    Reg({"HostReduceScatterSequenceMeshRHD", HCCL_CMD_REDUCE_SCATTER, HALG_RS_SEQ_MESH_RHD, "sequence", {"RHD", "Mesh"}, AlgoType::HD_R, 2, true, L, rs, false});
    Reg({"HostReduceScatterVSoleMesh", HCCL_CMD_REDUCE_SCATTER_V, HALG_RS_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, true, Two, rs, false});
    Reg({"HostReduceScatterVSoleRing", HCCL_CMD_REDUCE_SCATTER_V, HALG_RS_RING, "sole", {"Ring"}, AlgoType::RING, 1, true, P1, rs, false});
    Reg({"HostReduceScatterVSoleRHD", HCCL_CMD_REDUCE_SCATTER_V, HALG_RS_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, true, L, rs, false});
    Reg({"HostReduceScatterVSoleNHR", HCCL_CMD_REDUCE_SCATTER_V, HALG_RS_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, true, L, rs, false});
    // AllGather (+V)
    Reg({"HostAllGatherSoleMesh", HCCL_CMD_ALLGATHER, HALG_AG_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, false, Two, rs, true});
    Reg({"HostAllGatherSoleRing", HCCL_CMD_ALLGATHER, HALG_AG_RING, "sole", {"Ring"}, AlgoType::RING, 1, false, P1, rs, true});
    Reg({"HostAllGatherSoleRHD", HCCL_CMD_ALLGATHER, HALG_AG_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, false, L, rs, true});
    Reg({"HostAllGatherSoleNHR", HCCL_CMD_ALLGATHER, HALG_AG_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, false, L, rs, true});
    Reg({"HostAllGatherSequenceMeshNHRNHR", HCCL_CMD_ALLGATHER, HALG_AG_SEQ3_MESH_NHR_NHR, "sequence", {"Mesh", "NHR", "NHR"}, AlgoType::NHR, 3, false, L, rs, true});
    Reg({"HostAllGatherSequenceMeshNHR", HCCL_CMD_ALLGATHER, HALG_AG_SEQ_MESH_NHR, "sequence", {"Mesh", "NHR"}, AlgoType::NHR, 2, false, L, rs, true});
    Reg({"HostAllGatherSequenceMeshRing", HCCL_CMD_ALLGATHER, HALG_AG_SEQ_MESH_RING, "sequence", {"Mesh", "Ring"}, AlgoType::RING, 2, false, P1, rs, true});
    Reg({"HostAllGatherSequenceMeshRHD", HCCL_CMD_ALLGATHER, HALG_AG_SEQ_MESH_RHD, "sequence", {"Mesh", "RHD"}, AlgoType::HD_R, 2, false, L, rs, true});
    Reg({"HostAllGatherVSoleMesh", HCCL_CMD_ALLGATHER_V, HALG_AG_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, false, Two, rs, true});
    Reg({"HostAllGatherVSoleRing", HCCL_CMD_ALLGATHER_V, HALG_AG_RING, "sole", {"Ring"}, AlgoType::RING, 1, false, P1, rs, true});
    Reg({"HostAllGatherVSoleRHD", HCCL_CMD_ALLGATHER_V, HALG_AG_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, false, L, rs, true});
    Reg({"HostAllGatherVSoleNHR", HCCL_CMD_ALLGATHER_V, HALG_AG_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, false, L, rs, true});
    // Broadcast / Reduce / Scatter
    Reg({"HostBroadcastSoleMeshOneShot", HCCL_CMD_BROADCAST, HALG_BCAST_MESH_ONESHOT, "sole", {"MeshOneShot"}, AlgoType::ONESHOT, 1, false, Two, full, true});
    Reg({"HostBroadcastSoleMeshTwoShot", HCCL_CMD_BROADCAST, HALG_BCAST_MESH_TWOSHOT, "sole", {"MeshTwoShot"}, AlgoType::MESH, 1, false, Three, ar, true});
    Reg({"HostBroadcastSoleNHR", HCCL_CMD_BROADCAST, HALG_BCAST_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, false, L, ar, true});
    Reg({"HostBroadcastSoleRing", HCCL_CMD_BROADCAST, HALG_BCAST_RING, "sole", {"Ring"}, AlgoType::RING, 1, false, P1, ar, true});
    Reg({"HostBroadcastSoleRHD", HCCL_CMD_BROADCAST, HALG_BCAST_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, false, L, ar, true});
    Reg({"HostReduceSoleMeshOneShot", HCCL_CMD_REDUCE, HALG_REDUCE_MESH_ONESHOT, "sole", {"MeshOneShot"}, AlgoType::ONESHOT, 1, true, Two, full, true});
    Reg({"HostReduceSoleMeshTwoShot", HCCL_CMD_REDUCE, HALG_REDUCE_MESH_TWOSHOT, "sole", {"MeshTwoShot"}, AlgoType::MESH, 1, true, Three, ar, false});
    Reg({"HostReduceSoleNHR", HCCL_CMD_REDUCE, HALG_REDUCE_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, true, L, ar, false});
    Reg({"HostReduceSoleRing", HCCL_CMD_REDUCE, HALG_REDUCE_RING, "sole", {"Ring"}, AlgoType::RING, 1, true, P1, ar, false});
    Reg({"HostReduceSoleRHD", HCCL_CMD_REDUCE, HALG_REDUCE_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, true, L, ar, false});
    Reg({"HostScatterSoleMesh", HCCL_CMD_SCATTER, HALG_SCATTER_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, false, Two, rs, true});
    Reg({"HostScatterSoleRing", HCCL_CMD_SCATTER, HALG_SCATTER_RING, "sole", {"Ring"}, AlgoType::RING, 1, false, P1, one, true});
    // AlltoAll family
    for (HcclCMDType op : {HCCL_CMD_ALLTOALL, HCCL_CMD_ALLTOALLV, HCCL_CMD_ALLTOALLVC}) {
        const char* base = op == HCCL_CMD_ALLTOALL ? "HostAlltoAll" : op == HCCL_CMD_ALLTOALLV ? "HostAlltoAllV" : "HostAlltoAllVC";
        static std::vector<std::string> keep;
        keep.push_back(std::string(base) + "SoleMesh");
        Reg({keep.back().c_str(), op, HALG_A2A_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, false, Two, rs, true});
        keep.push_back(std::string(base) + "SolePairwise");
        Reg({keep.back().c_str(), op, HALG_A2A_PAIRWISE, "sole", {"Pairwise"}, AlgoType::PAIRWISE, 1, false, P1, rs, true});
        // one peer at a time through the staging buffer (every byte is copied twice): never the automatic choice
        keep.push_back(std::string(base) + "SerialSoleMesh");
        Reg({keep.back().c_str(), op, HALG_A2A_SERIAL, "serial", {"Mesh"}, AlgoType::SERIAL, 1, false, TwoP1, ar, true});
    }
    // Concurrent, Pipeline, Nonuniform Bruck, hierarchical and tree executors (host_executors.cc).  Their step counts
    // carry one extra step for the second queue or stage, so that automatic selection keeps the plain forms on ties.
    auto TwoL1 = [](double p) { return 2 * Log2Ceil(p) + 1; };
    auto L1 = [](double p) { return Log2Ceil(p) + 1; };
    auto Four = [](double) { return 4.0; };
    auto Five = [](double) { return 5.0; };
    auto TwoL2 = [](double p) { return 2 * Log2Ceil(p) + 2; };
    Reg({"HostAllReduceConcurrentMeshNHR", HCCL_CMD_ALLREDUCE, HALG_AR_CONCURRENT_MESH_NHR, "concurrent", {"Mesh", "NHR"}, AlgoType::CONCURRENT, 1, true, TwoL, ar, false});
    Reg({"HostReduceScatterConcurrentMeshNHR", HCCL_CMD_REDUCE_SCATTER, HALG_RS_CONCURRENT_MESH_NHR, "concurrent", {"Mesh", "NHR"}, AlgoType::CONCURRENT, 1, true, L, rs, false});
    Reg({"HostAllReduceSequence2DieMeshMesh", HCCL_CMD_ALLREDUCE, HALG_AR_SEQ_2DIE_MESH_MESH, "sequence2die", {"Mesh2Die", "Mesh2Die"}, AlgoType::TWO_DIE, 1, true, Four, ar, false});
    Reg({"HostAllReduceSoleMeshConcur", HCCL_CMD_ALLREDUCE, HALG_AR_SOLE_MESH_CONCUR, "twoshotsole", {"MeshConcur", "MeshConcur"}, AlgoType::MESH_CONCUR, 1, true, Four, ar, false});
    for (HcclCMDType op : {HCCL_CMD_ALLTOALL, HCCL_CMD_ALLTOALLV, HCCL_CMD_ALLTOALLVC}) {
        static std::vector<std::string> keepConcur;
        keepConcur.push_back(std::string(op == HCCL_CMD_ALLTOALL ? "HostAlltoAll" : op == HCCL_CMD_ALLTOALLV ? "HostAlltoAllV" : "HostAlltoAllVC") + "ConcurrentMeshMesh");
        Reg({keepConcur.back().c_str(), op, HALG_A2A_CONCURRENT_MESH_MESH, "concurrent", {"Mesh", "Mesh"}, AlgoType::CONCURRENT, 1, false, Three, rs, true});
    }
    Reg({"HostScatterConcurrentMeshMesh", HCCL_CMD_SCATTER, HALG_SCATTER_CONCURRENT_MESH_MESH, "concurrent", {"Mesh", "Mesh"}, AlgoType::CONCURRENT, 1, false, Three, rs, true});
    Reg({"HostBroadcastConcurrentMeshNHR", HCCL_CMD_BROADCAST, HALG_BCAST_CONCURRENT_MESH_NHR, "concurrent", {"Mesh", "NHR"}, AlgoType::CONCURRENT, 1, false, L1, ar, true});
    Reg({"HostReduceConcurrentMeshNHR", HCCL_CMD_REDUCE, HALG_REDUCE_CONCURRENT_MESH_NHR, "concurrent", {"Mesh", "NHR"}, AlgoType::CONCURRENT, 1, true, L1, ar, false});
    Reg({"HostAllGatherConcurrentMeshNHR", HCCL_CMD_ALLGATHER, HALG_AG_CONCURRENT_MESH_NHR, "concurrent", {"Mesh", "NHR"}, AlgoType::CONCURRENT, 1, false, L, rs, true});
    // three levels first: on a topology with pods it wins the tie with the two-level form, elsewhere it is filtered
    Reg({"HostAllReducePipelineMeshNHRNHR", HCCL_CMD_ALLREDUCE, HALG_AR_PIPELINE3_MESH_NHR_NHR, "pipeline", {"Mesh", "NHR", "NHR"}, AlgoType::OMNIPIPE, 3, true, TwoL1, ar, false});
    Reg({"HostAllReducePipelineMeshNHR", HCCL_CMD_ALLREDUCE, HALG_AR_PIPELINE_MESH_NHR, "pipeline", {"Mesh", "NHR"}, AlgoType::OMNIPIPE, 2, true, TwoL1, ar, false});
    Reg({"HostAllGatherPipelineMeshMeshMesh", HCCL_CMD_ALLGATHER, HALG_AG_PIPELINE3_MESH_MESH_MESH, "pipeline", {"Mesh", "Mesh", "Mesh"}, AlgoType::OMNIPIPE, 3, false, Four, rs, true});
    Reg({"HostReduceScatterPipelineMeshMeshMesh", HCCL_CMD_REDUCE_SCATTER, HALG_RS_PIPELINE3_MESH_MESH_MESH, "pipeline", {"Mesh", "Mesh", "Mesh"}, AlgoType::OMNIPIPE, 3, true, Four, rs, false});
    Reg({"HostAllGatherPipelineMeshMesh", HCCL_CMD_ALLGATHER, HALG_AG_PIPELINE_MESH_MESH, "pipeline", {"Mesh", "Mesh"}, AlgoType::OMNIPIPE, 2, false, Four, rs, true});
    Reg({"HostReduceScatterPipelineMeshMesh", HCCL_CMD_REDUCE_SCATTER, HALG_RS_PIPELINE_MESH_MESH, "pipeline", {"Mesh", "Mesh"}, AlgoType::OMNIPIPE, 2, true, Four, rs, false});
    Reg({"HostBroadcastPipelineMeshMesh", HCCL_CMD_BROADCAST, HALG_BCAST_PIPELINE_MESH_MESH, "pipeline", {"Mesh", "Mesh"}, AlgoType::OMNIPIPE, 2, false, Four, ar, true});
    Reg({"HostAllGatherParallelMeshMesh", HCCL_CMD_ALLGATHER, HALG_AG_PARALLEL_MESH_MESH, "parallel", {"Mesh", "Mesh"}, AlgoType::PIPELINE, 2, false, Four, rs, true});
    Reg({"HostReduceScatterParallelMeshMesh", HCCL_CMD_REDUCE_SCATTER, HALG_RS_PARALLEL_MESH_MESH, "parallel", {"Mesh", "Mesh"}, AlgoType::PIPELINE, 2, true, Four, rs, false});
    Reg({"HostBroadcastParallelMeshMesh", HCCL_CMD_BROADCAST, HALG_BCAST_PARALLEL_MESH_MESH, "parallel", {"Mesh", "Mesh"}, AlgoType::PIPELINE, 2, false, Four, ar, true});
    Reg({"HostScatterParallelMeshMesh", HCCL_CMD_SCATTER, HALG_SCATTER_PARALLEL_MESH_MESH, "parallel", {"Mesh", "Mesh"}, AlgoType::PIPELINE, 2, false, Five, rs, true});
    Reg({"HostReduceParallelMeshNHR", HCCL_CMD_REDUCE, HALG_REDUCE_PARALLEL_MESH_NHR, "parallel", {"Mesh", "NHR"}, AlgoType::PIPELINE, 2, true, TwoL2, ar, false});
    Reg({"HostAllGatherVPipelineMeshMesh", HCCL_CMD_ALLGATHER_V, HALG_AG_PIPELINE_MESH_MESH, "pipeline", {"Mesh", "Mesh"}, AlgoType::OMNIPIPE, 2, false, Four, rs, true});
    Reg({"HostReducePipelineMeshNHR", HCCL_CMD_REDUCE, HALG_REDUCE_PIPELINE_MESH_NHR, "pipeline", {"Mesh", "NHR"}, AlgoType::OMNIPIPE, 2, true, TwoL2, ar, false});
    Reg({"HostScatterPipelineMeshMesh", HCCL_CMD_SCATTER, HALG_SCATTER_PIPELINE_MESH_MESH, "pipeline", {"Mesh", "Mesh"}, AlgoType::OMNIPIPE, 2, false, Five, rs, true});
    Reg({"HostAllGatherSoleMeshZAxisDetour", HCCL_CMD_ALLGATHER, HALG_AG_MESH_DETOUR, "sole", {"MeshZAxisDetour"}, AlgoType::DETOUR, 1, false, Two, rs, true});
    Reg({"HostReduceScatterSoleMeshZAxisDetour", HCCL_CMD_REDUCE_SCATTER, HALG_RS_MESH_DETOUR, "sole", {"MeshZAxisDetour"}, AlgoType::DETOUR, 1, true, Two, rs, false});
    Reg({"HostScatterSoleMeshZAxisDetour", HCCL_CMD_SCATTER, HALG_SCATTER_MESH_DETOUR, "sole", {"MeshZAxisDetour"}, AlgoType::DETOUR, 1, false, Two, rs, true});
    Reg({"HostAllGatherSoleNB", HCCL_CMD_ALLGATHER, HALG_AG_NB, "sole", {"NB"}, AlgoType::NB, 1, false, L1, rs, true});
    Reg({"HostBroadcastSoleNB", HCCL_CMD_BROADCAST, HALG_BCAST_NB, "sole", {"NB"}, AlgoType::NB, 1, false, L1, ar, true});
    Reg({"HostScatterSoleNB", HCCL_CMD_SCATTER, HALG_SCATTER_NB, "sole", {"NB"}, AlgoType::NB, 1, false, L1, one, true});
    Reg({"HostBroadcastSequenceMeshNHR", HCCL_CMD_BROADCAST, HALG_BCAST_SEQ_MESH_NHR, "sequence", {"Mesh", "NHR"}, AlgoType::NHR, 2, false, TwoL1, ar, true});
    Reg({"HostReduceSequenceMeshNHR", HCCL_CMD_REDUCE, HALG_REDUCE_SEQ_MESH_NHR, "sequence", {"Mesh", "NHR"}, AlgoType::NHR, 2, true, TwoL1, ar, false});
    Reg({"HostScatterSequenceMeshMesh", HCCL_CMD_SCATTER, HALG_SCATTER_SEQ_MESH_MESH, "sequence", {"Mesh", "Mesh"}, AlgoType::HIER, 2, false, Four, rs, true});
    Reg({"HostBarrierSequenceMeshNHR", HCCL_CMD_BARRIER, HALG_BARRIER_SEQ_MESH_NHR, "sequence", {"Mesh", "NHR"}, AlgoType::HIER, 2, false, TwoL1, [](double) { return 0.0; }, true});
    Reg({"HostAllReduceTree", HCCL_CMD_ALLREDUCE, HALG_AR_TREE, "tree", {"Tree"}, AlgoType::TREE, 1, true, TwoL1, ar, false});
    for (HcclCMDType op : {HCCL_CMD_ALLTOALL, HCCL_CMD_ALLTOALLV, HCCL_CMD_ALLTOALLVC}) {
        static std::vector<std::string> keepHier;
        keepHier.push_back(std::string(op == HCCL_CMD_ALLTOALL ? "HostAlltoAll" : op == HCCL_CMD_ALLTOALLV ? "HostAlltoAllV" : "HostAlltoAllVC") + "HierMeshMesh");
        Reg({keepHier.back().c_str(), op, HALG_A2A_HIER, "hier", {"Mesh", "Mesh"}, AlgoType::HIER, 2, false, Four, ar, true});
    }
    // point to point and barrier
    Reg({"HostSendSoleMesh", HCCL_CMD_SEND, HALG_P2P_DIRECT, "sole", {"Direct"}, AlgoType::MESH, 1, false, one, one, true});
    Reg({"HostRecvSoleMesh", HCCL_CMD_RECEIVE, HALG_P2P_DIRECT, "sole", {"Direct"}, AlgoType::MESH, 1, false, one, one, true});
    Reg({"HostBatchSendRecvSoleMesh", HCCL_CMD_BATCH_SEND_RECV, HALG_P2P_DIRECT, "sole", {"Direct"}, AlgoType::MESH, 1, false, one, one, true});
    Reg({"HostBarrierSoleMesh", HCCL_CMD_BARRIER, HALG_BARRIER_MESH, "sole", {"Mesh"}, AlgoType::MESH, 1, false, one, [](double) { return 0.0; }, true});
    Reg({"HostBarrierSoleNHR", HCCL_CMD_BARRIER, HALG_BARRIER_NHR, "sole", {"NHR"}, AlgoType::NHR, 1, false, L, [](double) { return 0.0; }, true});
    Reg({"HostBarrierSoleRHD", HCCL_CMD_BARRIER, HALG_BARRIER_RHD, "sole", {"RHD"}, AlgoType::HD_R, 1, false, L, [](double) { return 0.0; }, true});
}

}  // namespace hccl

using namespace hccl;

extern "C" {

HcclResult HcclTestHostDropPosts(HcclComm comm, uint32_t count)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->hostComm) return HCCL_E_NOT_SUPPORT;
    c->hostComm->world->DropPosts(c->hostComm->rank, count);
    return HCCL_SUCCESS;
}

HcclResult HcclTestHostRecoveries(HcclComm comm, uint64_t* count)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(count);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->hostComm) return HCCL_E_NOT_SUPPORT;
    *count = c->hostComm->world->recoveries();
    return HCCL_SUCCESS;
}

// Topology self-test entry: the model a topology literal gives `rank`, the groups of the requested match
// (0 one level, 1 two levels, 2 three levels), and the serialisation guards (a round trip restores the model, a
// damaged or truncated blob is refused).
HcclResult HcclDebugTopo(const char* topoJson, uint32_t nRanks, uint32_t rank, int matchKind, char* text, uint32_t capacity)
{
    CHK_PTR_NULL(text);
    TopoMeta meta;
    std::string err;
    if (nRanks == 0 || rank >= nRanks || matchKind < 0 || matchKind > 3) return HCCL_E_PARA;
    if (!ParseTopoMeta(topoJson, nRanks, &meta, &err)) { snprintf(text, capacity, "error: %s", err.c_str()); return HCCL_SUCCESS; }
    TopoInfo t;
    CHK_RET(BuildTopoFromMeta(meta, rank, &t));
    std::ostringstream os;
    os << t.Summary() << "\n";
    os << "server " << t.serverOf[rank] << " pod " << t.podOf[rank] << " local " << t.localOf[rank] << " symmetric " << t.symmetric << " level1Nhr " << t.level1Nhr << "\n";
    AlgHierarchy h;
    const HcclResult mr = MatchTopo(t, (TopoMatchKind)matchKind, &h);
    if (mr != HCCL_SUCCESS) os << "match: " << ResultString(mr) << "\n";
    else {
        for (uint32_t l = 0; l < h.levels(); ++l) {
            os << "level " << l << ":";
            for (auto& g : h.infos[l]) {
                os << " [";
                for (size_t i = 0; i < g.size(); ++i) os << (i ? "," : "") << g[i];
                os << "]";
            }
            os << "\n";
        }
    }
    std::vector<uint8_t> blob = t.Serialize();
    TopoInfo back;
    const bool ok = TopoInfo::Deserialize(blob, &back) && back.nRanks == t.nRanks && back.serverOf == t.serverOf && back.localOf == t.localOf && back.symmetric == t.symmetric;
    std::vector<uint8_t> bad = blob;
    bad[bad.size() / 2] ^= 0x5A;
    std::vector<uint8_t> cut(blob.begin(), blob.begin() + (long)(blob.size() / 2));
    TopoInfo junk;
    os << "roundtrip " << ok << " damaged " << TopoInfo::Deserialize(bad, &junk) << " truncated " << TopoInfo::Deserialize(cut, &junk) << "\n";
    snprintf(text, capacity, "%s", os.str().c_str());
    return HCCL_SUCCESS;
}

// Verifier self-test entry: checks a trace written as text.  First line "ranks <n> op <allreduce|allgather|
// reducescatter|reduce|scatter|alltoall> count <elements> [root <r>]" (fp32, sum); then one task per line:
//   <rank> <queue> copy|reduce <dstRank>:<in|out|scr>:<byteOffset> <srcRank>:<in|out|scr>:<byteOffset> <bytes>
//   <rank> <queue> post|wait <peer> <notifyIdx>
HcclResult HcclDebugVerifyTrace(const char* script, char* report, uint32_t capacity)
{
    CHK_PTR_NULL(script); CHK_PTR_NULL(report);
    std::istringstream is(script);
    std::string word, opName;
    uint32_t n = 0, root = 0;
    uint64_t count = 0;
    std::string header;
    std::getline(is, header);
    std::istringstream hs(header);
    while (hs >> word) {
        if (word == "ranks") hs >> n;
        else if (word == "op") hs >> opName;
        else if (word == "count") hs >> count;
        else if (word == "root") hs >> root;
    }
    static const std::map<std::string, HcclCMDType> kOps = {{"allreduce", HCCL_CMD_ALLREDUCE}, {"allgather", HCCL_CMD_ALLGATHER},
        {"reducescatter", HCCL_CMD_REDUCE_SCATTER}, {"reduce", HCCL_CMD_REDUCE}, {"scatter", HCCL_CMD_SCATTER}, {"alltoall", HCCL_CMD_ALLTOALL}};
    auto it = kOps.find(opName);
    if (n == 0 || n > 64 || count == 0 || it == kOps.end() || root >= n) return HCCL_E_PARA;
    HostOpDesc d;
    d.op = it->second; d.dtype = HCCL_DATA_TYPE_FP32; d.redOp = HCCL_REDUCE_SUM; d.count = count; d.root = root;
    const uint64_t unit = count * 4;
    const bool inWide = d.op == HCCL_CMD_REDUCE_SCATTER || d.op == HCCL_CMD_SCATTER || d.op == HCCL_CMD_ALLTOALL;
    const bool outWide = d.op == HCCL_CMD_ALLGATHER || d.op == HCCL_CMD_ALLTOALL;
    auto mem = [&](const std::string& text, Mem* m) {
        unsigned r = 0;
        char buf[8] = {0};
        unsigned long long off = 0;
        if (sscanf(text.c_str(), "%u:%3[a-z]:%llu", &r, buf, &off) != 3 || r >= n) return false;
        const std::string b(buf);
        m->rank = r;
        m->off = off;
        m->buf = b == "in" ? BufKind::INPUT : b == "out" ? BufKind::OUTPUT : BufKind::SCRATCH;
        return b == "in" || b == "out" || b == "scr";
    };
    std::vector<std::vector<Task>> tasks(n);
    std::string line;
    while (std::getline(is, line)) {
        std::istringstream ls(line);
        uint32_t rank, queue;
        std::string kind;
        if (!(ls >> rank >> queue >> kind)) continue;      // blank line
        if (rank >= n) return HCCL_E_PARA;
        Task t{};
        t.rank = rank;
        t.queue = queue;
        if (kind == "post" || kind == "wait") {
            if (!(ls >> t.peer >> t.notifyIdx) || t.peer >= n || t.notifyIdx >= HostWorld::kNotifyIdx) return HCCL_E_PARA;
            t.kind = kind == "post" ? TaskKind::POST : TaskKind::WAIT;
        } else if (kind == "copy" || kind == "reduce") {
            std::string dst, src;
            if (!(ls >> dst >> src >> t.bytes) || !mem(dst, &t.dst) || !mem(src, &t.src)) return HCCL_E_PARA;
            const bool local = t.dst.rank == rank && t.src.rank == rank, reads = t.dst.rank == rank;
            if (kind == "copy") t.kind = local ? TaskKind::LOCAL_COPY : reads ? TaskKind::READ : TaskKind::WRITE;
            else t.kind = local ? TaskKind::LOCAL_REDUCE : reads ? TaskKind::READ_REDUCE : TaskKind::WRITE_REDUCE;
        } else {
            return HCCL_E_PARA;
        }
        tasks[rank].push_back(t);
    }
    TopoMeta meta;
    std::string err;
    if (!ParseTopoMeta(nullptr, n, &meta, &err)) return HCCL_E_INTERNAL;
    HostWorld world(n, meta, 1 << 20, 1000000000ull);
    const VerifyReport rep = world.VerifyTasks(d, unit * (inWide ? n : 1), unit * (outWide ? n : 1), tasks);
    snprintf(report, capacity, "%s", rep.Text().c_str());
    return HCCL_SUCCESS;
}

HcclResult HcclHostTraceBegin(HcclComm comm)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->hostComm) return HCCL_E_NOT_SUPPORT;
    c->hostComm->world->TraceBegin();
    return HCCL_SUCCESS;
}

HcclResult HcclHostTraceVerify(HcclComm comm, char* report, uint32_t capacity)
{
    CHK_PTR_NULL(comm);
    CommImpl* c = static_cast<CommImpl*>(comm);
    if (!c->hostComm) return HCCL_E_NOT_SUPPORT;
    VerifyReport rep = c->hostComm->world->Verify();
    if (report && capacity) snprintf(report, capacity, "%s", rep.Text().c_str());
    return rep.ok ? HCCL_SUCCESS : HCCL_E_INTERNAL;
}

}  // extern "C"
