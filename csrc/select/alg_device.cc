// Registration of the device-engine algorithms with their attributes and cost
// coefficients.  One entry per (engine, op, strategy, template); the executor is
// "sole" for all of them because one NVSwitch box is a single level-0 mesh
// (reference equivalents: AivAllReduceSoleMeshOneShot / AivAllReduceSoleMeshTwoShot
// ins_v2_all_reduce_sole_executor.cc:459,481, CcuMSAllReduceSoleMesh :548, and
// the Sole/Mesh entries of the other operators listed with REGISTER_EXEC_V2).
#include <algorithm>
#include "selector.h"
#include "../core/config.h"
#include "../kernels/dev_types.h"
#include "../kernels/launch.h"

namespace hccl {
namespace {

constexpr uint64_t Bit(HcclDataType t) { return 1ull << (int)t; }
constexpr uint64_t kReduceTypes = Bit(HCCL_DATA_TYPE_INT8) | Bit(HCCL_DATA_TYPE_INT16) | Bit(HCCL_DATA_TYPE_INT32) |
                                  Bit(HCCL_DATA_TYPE_INT64) | Bit(HCCL_DATA_TYPE_UINT64) | Bit(HCCL_DATA_TYPE_FP16) |
                                  Bit(HCCL_DATA_TYPE_BFP16) | Bit(HCCL_DATA_TYPE_FP32) | Bit(HCCL_DATA_TYPE_FP64);
constexpr uint64_t kNvlsTypes = Bit(HCCL_DATA_TYPE_FP16) | Bit(HCCL_DATA_TYPE_BFP16) | Bit(HCCL_DATA_TYPE_FP32);
constexpr uint64_t kFp8Types = Bit(HCCL_DATA_TYPE_FP8E4M3) | Bit(HCCL_DATA_TYPE_FP8E5M2);
constexpr uint32_t kMeshShapes = (1u << (int)Level0Shape::MESH_1D) | (1u << (int)Level0Shape::SINGLE);

double UsPerByte(double gbs) { return 1.0 / (gbs * 1e3); }

// Common pieces of the coefficient sets.
struct M {
    const LinkModel& lm;
    double p;
    bool stageIn, stageOut;
    M(const TopoInfo& t, const OpDesc& o) : lm(GlobalLinkModel()), p((double)t.nRanks), stageIn(!o.inRegistered || !o.aligned16), stageOut(!o.aligned16) {}
    double link() const { return UsPerByte(lm.p2pGBs); }
    double nvls() const { return UsPerByte(lm.nvlsGBs); }
    double nvlsReduceOut() const { return UsPerByte(lm.nvlsReduceOutGBs); }
    double nvlsStore() const { return UsPerByte(lm.nvlsStoreGBs); }
    double copy() const { return UsPerByte(lm.localCopyGBs); }
};

AlgEntry Base(const char* name, HcclCMDType op, HcclCommEngine eng, const char* templ, int devAlg, AlgoType family)
{
    AlgEntry e;
    e.name = name;
    e.op = op;
    e.engine = eng;
    e.executor = "sole";
    e.templates = {templ};
    e.devAlg = devAlg;
    e.family = family;
    e.attrs.level0Shapes = kMeshShapes;
    e.attrs.maxRankSize = kMaxDevRanks;
    e.attrs.needsDeviceP2p = true;
    return e;
}

// Flag-in-data exchanges move one pair's block through one line slot of kLLMaxPayload payload bytes.
bool PairFitsLLSlot(const OpDesc& o, const TopoInfo& t, std::string* why)
{
    const uint64_t pair = o.bytes / std::max<uint64_t>(1, t.nRanks);
    if (pair > kLLMaxPayload) { if (why) *why = "op: a pair's block exceeds the line slot"; return false; }
    return true;
}

void RegisterAll()
{
    AlgRegistry& R = AlgRegistry::Instance();
    // ---------------- AllReduce
    {
        AlgEntry e = Base("P2pAllReduceSoleMeshLL", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshLL", DALG_AR_LL, AlgoType::LL);
        e.attrs.dtypeMask = kReduceTypes;
        // every rank writes the whole message (doubled by the flags) to every peer, so the form stops paying off around
        // 64 KiB, where the barrier forms catch up
        e.attrs.maxBytes = 64 * 1024;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            // every rank writes 2x the payload to each peer; latency-bound: modelled without a utilisation curve
            c.B = 2.0 * (m.p - 1) * m.link() + 2.0 * m.p * m.copy();
            c.C = m.lm.launchUs + m.lm.llHopUs;
            c.net = NetType::LOCAL;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pAllReduceSoleMeshOneShot", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshOneShot", DALG_AR_ONESHOT, AlgoType::ONESHOT);
        e.attrs.dtypeMask = kReduceTypes;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) * m.link();
            c.ratio = 1.0;
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pAllReduceSoleMeshTwoShot", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshTwoShot", DALG_AR_TWOSHOT, AlgoType::TWOSHOT);
        e.attrs.dtypeMask = kReduceTypes;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + (m.stageOut ? m.copy() : 0) + m.copy() / m.p;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("NvlsAllReduceSoleMesh", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_NVLS, "Mesh", DALG_AR_NVLS, AlgoType::NVLS);
        e.attrs.dtypeMask = kNvlsTypes;
        e.attrs.supportProd = false;
        e.attrs.supportMaxMin = false;
        e.attrs.needsNvls = true;
        // the switch's reduction order is not specified: excluded under deterministic / strict
        e.attrs.orderPreserved = false;
        e.attrs.deterministic = false;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            // every rank reduces 1/p of the message through the switch and multicasts it; its port carries the message once
            c.A = std::max((m.nvlsReduceOut() + m.nvlsStore()) / m.p, (1.0 + 1.0 / m.p) * m.nvls());
            c.ratio = 1.0 / m.p;
            c.net = NetType::NVLS_SWITCH;
            // the switch reads and writes through multicast aliases: anything without one is staged through the slab
            c.B = ((m.stageIn || !o.inMulticast) ? m.copy() : 0) + ((!o.outMulticast || !o.aligned16) ? m.copy() : 0);
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- ReduceScatter (+V)
    for (HcclCMDType op : {HCCL_CMD_REDUCE_SCATTER, HCCL_CMD_REDUCE_SCATTER_V}) {
        const bool v = op == HCCL_CMD_REDUCE_SCATTER_V;
        {
            AlgEntry e = Base(v ? "P2pReduceScatterVSoleMesh" : "P2pReduceScatterSoleMesh", op, HCCL_ENGINE_P2P, "Mesh", DALG_RS_PULL, AlgoType::MESH);
            e.attrs.dtypeMask = kReduceTypes | (v ? 0 : kFp8Types);
            e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
                M m(t, o);
                CostCoeff c;
                c.A = (m.p - 1) / m.p * m.link();
                c.ratio = 1.0 / m.p;
                c.B = m.stageIn ? m.copy() : 0;
                c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
                return std::vector<CostCoeff>{c};
            };
            R.Register(e);
        }
        {
            AlgEntry e = Base(v ? "NvlsReduceScatterVSoleMesh" : "NvlsReduceScatterSoleMesh", op, HCCL_ENGINE_NVLS, "Mesh", DALG_RS_NVLS, AlgoType::NVLS);
            e.attrs.dtypeMask = kNvlsTypes;
            e.attrs.supportProd = false;
            e.attrs.supportMaxMin = false;
            e.attrs.needsNvls = true;
            e.attrs.orderPreserved = false;
            e.attrs.deterministic = false;
            e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
                M m(t, o);
                CostCoeff c;
                c.A = m.nvlsReduceOut() / m.p;      // each rank receives its reduced share once; peers feed the switch in parallel
                c.ratio = 1.0 / m.p;
                c.net = NetType::NVLS_SWITCH;
                c.B = (m.stageIn || !o.inMulticast) ? m.copy() : 0;
                c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
                // the switch still has to pull (p-1)/p of the input out of every GPU, at the rate of a port (measured 623 GB/s
                // of egress at 1 GiB on 8 GPUs), and a staged input is copied before any of that starts
                c.D = ((m.p - 1) / m.p * m.link() + c.B) * (double)o.bytes;
                // An ordinary input has to be copied into the slab before the switch can read it.  Measured at 8 GPUs next to
                // the push form, which lands the blocks without that pass: 38 / 55 / 137 / 521 / 1953 us against 37 / 46 /
                // 114 / 441 / 1705 us at 4 / 16 / 64 / 256 / 1024 MiB.  So this form is never priced below 1.05 x the push
                // form's own estimate for such an input.
                if (!o.inRegistered && o.aligned16) {
                    const double util = LinkUtilisation(NetType::MESH_P2P, (double)o.bytes / m.p, HCCL_ENGINE_P2P, (int)t.nRanks);
                    const double push = ((m.p - 1) / m.p * m.link() / util + 0.25 * m.copy()) * (double)o.bytes + m.lm.launchUs + m.lm.barrierUs;
                    c.D = std::max(c.D, 1.05 * push);
                }
                return std::vector<CostCoeff>{c};
            };
            R.Register(e);
        }
    }
    // ---------------- AllGather (+V)
    for (HcclCMDType op : {HCCL_CMD_ALLGATHER, HCCL_CMD_ALLGATHER_V}) {
        const bool v = op == HCCL_CMD_ALLGATHER_V;
        {
            AlgEntry e = Base(v ? "P2pAllGatherVSoleMesh" : "P2pAllGatherSoleMesh", op, HCCL_ENGINE_P2P, "Mesh", DALG_AG_PULL, AlgoType::MESH);
            e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
                M m(t, o);
                CostCoeff c;
                c.A = (m.p - 1) / m.p * m.link();
                c.ratio = 1.0 / m.p;
                c.B = (m.stageIn ? m.copy() / m.p : 0) + m.copy() / m.p;
                c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
                return std::vector<CostCoeff>{c};
            };
            R.Register(e);
        }
        if (!v) {
            AlgEntry e = Base("P2pAllGatherSoleMeshLL", op, HCCL_ENGINE_P2P, "MeshLL", DALG_AG_LL, AlgoType::LL);
            e.attrs.opCustomCheck = [](const OpDesc& o, const TopoInfo& t, std::string* why) {
                if (o.bytes / t.nRanks > kLLMaxPayload) { *why = "op: per-rank block exceeds the LL slot"; return false; }
                return true;
            };
            e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
                M m(t, o);
                CostCoeff c;
                c.B = 2.0 * (m.p - 1) / m.p * m.link() + 2.0 * m.copy();
                c.C = m.lm.launchUs + m.lm.llHopUs;
                c.net = NetType::LOCAL;
                return std::vector<CostCoeff>{c};
            };
            R.Register(e);
        }
    }
    // ---------------- small-message forms: flag-in-data lines, one latency, no barrier
    {
        AlgEntry e = Base("P2pReduceScatterSoleMeshLL", HCCL_CMD_REDUCE_SCATTER, HCCL_ENGINE_P2P, "MeshLL", DALG_RS_LL, AlgoType::LL);
        e.attrs.dtypeMask = kReduceTypes;
        e.attrs.maxBytes = 1024 * 1024;           // whole input; a pair moves 1/p of it (measured at 8 ranks: ahead of the switch form up to here)
        e.attrs.opCustomCheck = PairFitsLLSlot;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.B = 2.0 * (m.p - 1) / m.p * m.link() + 2.0 * m.copy();
            c.C = m.lm.launchUs + m.lm.llHopUs;
            c.net = NetType::LOCAL;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pBroadcastSoleMeshLL", HCCL_CMD_BROADCAST, HCCL_ENGINE_P2P, "MeshLL", DALG_BCAST_LL, AlgoType::LL);
        e.attrs.maxBytes = 64 * 1024;             // the root writes the message (doubled by the flags) to every peer
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.B = 2.0 * (m.p - 1) * m.link() + 2.0 * m.copy();
            c.C = m.lm.launchUs + m.lm.llHopUs;
            c.net = NetType::LOCAL;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pAlltoAllSoleMeshLL", HCCL_CMD_ALLTOALL, HCCL_ENGINE_P2P, "MeshLL", DALG_A2A_LL, AlgoType::LL);
        // the pull form pays two barriers and a table exchange (42 us at 8 ranks whatever the size below 16 MiB), the
        // flag-in-data form one latency: it stays ahead as long as a pair's block fits a line slot
        e.attrs.maxBytes = 2 * 1024 * 1024;
        e.attrs.opCustomCheck = PairFitsLLSlot;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.B = 2.0 * (m.p - 1) / m.p * m.link() + 2.0 * m.copy();
            c.C = m.lm.launchUs + m.lm.llHopUs;
            c.net = NetType::LOCAL;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- Broadcast
    {
        AlgEntry e = Base("P2pBroadcastSoleMeshOneShot", HCCL_CMD_BROADCAST, HCCL_ENGINE_P2P, "MeshOneShot", DALG_BCAST_ONESHOT, AlgoType::ONESHOT);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) * m.link();    // the root's egress carries the message p-1 times
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pBroadcastSoleMeshTwoShot", HCCL_CMD_BROADCAST, HCCL_ENGINE_P2P, "MeshTwoShot", DALG_BCAST_TWOSHOT, AlgoType::TWOSHOT);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + m.copy() / m.p;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("NvlsBroadcastSoleMesh", HCCL_CMD_BROADCAST, HCCL_ENGINE_NVLS, "Mesh", DALG_BCAST_NVLS, AlgoType::NVLS);
        e.attrs.needsNvls = true;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = m.nvlsStore();
            c.net = NetType::NVLS_SWITCH;
            c.B = o.inMulticast && o.aligned16 ? 0 : m.copy();     // stored straight into a buffer with a multicast alias
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- Reduce
    {
        AlgEntry e = Base("P2pReduceSoleMeshOneShot", HCCL_CMD_REDUCE, HCCL_ENGINE_P2P, "MeshOneShot", DALG_REDUCE_ONESHOT, AlgoType::ONESHOT);
        e.attrs.dtypeMask = kReduceTypes;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) * m.link();
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pReduceSoleMeshTwoShot", HCCL_CMD_REDUCE, HCCL_ENGINE_P2P, "MeshTwoShot", DALG_REDUCE_TWOSHOT, AlgoType::TWOSHOT);
        e.attrs.dtypeMask = kReduceTypes;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- Scatter
    {
        AlgEntry e = Base("P2pScatterSoleMesh", HCCL_CMD_SCATTER, HCCL_ENGINE_P2P, "Mesh", DALG_SCATTER_PULL, AlgoType::MESH);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- AlltoAll family
    for (HcclCMDType op : {HCCL_CMD_ALLTOALL, HCCL_CMD_ALLTOALLV, HCCL_CMD_ALLTOALLVC}) {
        const char* name = op == HCCL_CMD_ALLTOALL ? "P2pAlltoAllSoleMesh" : (op == HCCL_CMD_ALLTOALLV ? "P2pAlltoAllVSoleMesh" : "P2pAlltoAllVCSoleMesh");
        AlgEntry e = Base(name, op, HCCL_ENGINE_P2P, "Mesh", DALG_A2A_PULL, AlgoType::MESH);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + m.copy() / m.p;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;          // two barriers and the read of the senders' offset tables
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- AlltoAllV whose size exchange and start barrier run on one block row per rank (the counts are
    // private to each rank, so every rank launches the full grid; here only the rows the data needs run barriers)
    {
        AlgEntry e = Base("P2pAlltoAllVSoleMeshLeader", HCCL_CMD_ALLTOALLV, HCCL_ENGINE_P2P, "MeshLeader", DALG_A2AV_LEADER, AlgoType::MESH);
        e.attrs.opCustomCheck = [](const OpDesc&, const TopoInfo&, std::string* why) {
            if (!GetEnvConfig().a2avLeader) { *why = "config: HCCL_A2AV_LEADER=0"; return false; }
            return true;
        };
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + m.copy() / m.p;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- reductions fused with a cast and a scale (only for calls that ask for one)
    {
        constexpr uint64_t kCastTypes = Bit(HCCL_DATA_TYPE_FP16) | Bit(HCCL_DATA_TYPE_BFP16) | Bit(HCCL_DATA_TYPE_FP32);
        AlgEntry e = Base("P2pAllReduceSoleMeshOneShotCast", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshOneShotCast", DALG_AR_ONESHOT_CAST, AlgoType::ONESHOT);
        e.attrs.dtypeMask = kCastTypes;
        e.attrs.castScale = true;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) * m.link();
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
        AlgEntry f = Base("P2pAllReduceSoleMeshTwoShotCast", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshTwoShotCast", DALG_AR_TWOSHOT_CAST, AlgoType::TWOSHOT);
        f.attrs.dtypeMask = kCastTypes;
        f.attrs.castScale = true;
        f.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + 2.0 * m.copy() / m.p;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(f);
        AlgEntry g = Base("P2pReduceScatterSoleMeshCast", HCCL_CMD_REDUCE_SCATTER, HCCL_ENGINE_P2P, "MeshCast", DALG_RS_CAST, AlgoType::MESH);
        g.attrs.dtypeMask = kCastTypes;
        g.attrs.castScale = true;
        g.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = m.stageIn ? m.copy() : 0;
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(g);
    }
    // ---------------- ring and halving-doubling templates on the device: neighbour / partner flags between the steps.
    // On one NVSwitch box the mesh forms move the same bytes in fewer steps, so the cost model only takes these when
    // HCCL_ALGO names them (ring, H-D_R) or a tuner prefers them; they are the level-1 candidates of a multi-box
    // topology.
    {
        AlgEntry e = Base("P2pReduceScatterSoleRing", HCCL_CMD_REDUCE_SCATTER, HCCL_ENGINE_P2P, "Ring", DALG_RS_RING, AlgoType::RING);
        e.attrs.dtypeMask = kReduceTypes;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() : 0) + 2.0 * (m.p - 1) / m.p * m.copy();
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs + (m.p - 1) * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
        AlgEntry f = Base("P2pAllGatherSoleRing", HCCL_CMD_ALLGATHER, HCCL_ENGINE_P2P, "Ring", DALG_AG_RING, AlgoType::RING);
        f.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = (m.stageIn ? m.copy() / m.p : 0) + 2.0 * m.copy();
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs + (m.p - 1) * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(f);
        AlgEntry g = Base("P2pAllReduceSoleRhd", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "Rhd", DALG_AR_RHD, AlgoType::HD_R);
        g.attrs.dtypeMask = kReduceTypes;
        g.attrs.powerOfTwoRanksOnly = true;
        g.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            double steps = 0;
            for (double q = 1; q < m.p; q *= 2) steps += 1;
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 0.5;
            c.B = (m.stageIn ? m.copy() : 0) + 3.0 * m.copy();
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs + 2.0 * steps * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(g);
    }
    // ---------------- switch multicast AllGather; Broadcast as scatter + switch AllGather
    {
        AlgEntry e = Base("NvlsAllGatherSoleMesh", HCCL_CMD_ALLGATHER, HCCL_ENGINE_NVLS, "Mesh", DALG_AG_NVLS, AlgoType::NVLS);
        e.attrs.needsNvls = true;
        e.attrs.needsAligned16 = true;
        e.attrs.opCustomCheck = [](const OpDesc& o, const TopoInfo& t, std::string* why) {
            if ((o.bytes / std::max<uint32_t>(1, t.nRanks)) % 16 != 0) { *why = "op: blocks are not a multiple of 16 bytes"; return false; }
            return true;
        };
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            // a port sends its block once and receives p - 1 blocks: bound by the same ingress as the pull form.  Priced a
            // little above it until a measurement on the box says otherwise (HCCL_ALGO="allgather=level0:nvls" picks it)
            c.A = std::max((m.p - 1) / m.p * m.link() * 1.03, m.nvlsStore() / m.p);
            c.ratio = 1.0 / m.p;
            c.B = m.copy() / m.p + (o.outMulticast ? 0 : m.copy());      // without a multicast alias the blocks are copied out of the slab
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
        AlgEntry f = Base("NvlsBroadcastSoleMeshScatter", HCCL_CMD_BROADCAST, HCCL_ENGINE_NVLS, "MeshScatter", DALG_BCAST_SCATTER_NVLS, AlgoType::NVLS);
        f.attrs.needsNvls = true;
        f.attrs.minBytes = 1024 * 1024;
        // a receiver's port takes multicast stores at about two thirds of the rate of peer reads (measured at 8 GPUs:
        // 485 GB/s of bus bandwidth at 1 GiB against 538 GB/s for the pipelined peer-read form, which has more steps and
        // only wins from 512 MiB up)
        f.attrs.maxBytes = 384ull << 20;
        // two ranks: the one receiver pulls half and is sent the other half through the switch, measured 0.72-0.86 of
        // NCCL from 8 MiB up where the plain pull of everything runs at 1.12
        f.attrs.opCustomCheck = [](const OpDesc&, const TopoInfo& t, std::string* why) {
            if (t.nRanks < 3) { *why = "topo: fewer than three ranks"; return false; }
            return true;
        };
        f.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            // the root's port carries (p - 1) / p of the message once; every port then multicasts 1 / p
            c.A = (m.p - 1) / m.p * m.link() + std::max(m.nvlsStore() / m.p, (m.p - 1) / m.p * m.nvls()) * 0.25;
            c.ratio = 1.0 / m.p;
            c.net = NetType::NVLS_SWITCH;
            c.B = (m.stageIn ? m.copy() : 0) + ((o.inMulticast && o.aligned16) ? 0 : m.copy());
            c.C = m.lm.launchUs + 2 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(f);
    }
    // ---------------- AlltoAll through the receivers' slabs: posted writes, one barrier, a local copy
    {
        AlgEntry e = Base("P2pAlltoAllSoleMeshPush", HCCL_CMD_ALLTOALL, HCCL_ENGINE_P2P, "MeshPush", DALG_A2A_PUSH, AlgoType::MESH);
        e.attrs.maxBytes = 64ull << 20;
        e.attrs.opCustomCheck = [](const OpDesc& o, const TopoInfo& t, std::string* why) {
            // both landing copies of all pairs' blocks must fit the stage-in region: about a quarter of the slab (the
            // executor checks the exact size and the selector only offers the form well inside it)
            const uint64_t pair = o.bytes / std::max<uint32_t>(1, t.nRanks);
            if ((pair + 16) * t.nRanks * 2 > o.stageInBytes) { *why = "op: the blocks do not fit the landing zone twice"; return false; }
            return true;
        };
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = 1.0 * m.copy();           // the landed blocks are copied out once, locally
            c.C = m.lm.launchUs + m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- Broadcast of large messages: pipelined scatter + AllGather over peer reads
    {
        AlgEntry e = Base("P2pBroadcastSoleMeshPipe", HCCL_CMD_BROADCAST, HCCL_ENGINE_P2P, "MeshPipe", DALG_BCAST_PIPE, AlgoType::PIPELINE);
        e.attrs.needsAligned16 = true;
        e.attrs.minBytes = 4ull << 20;
        e.attrs.opCustomCheck = [](const OpDesc& o, const TopoInfo& t, std::string* why) {
            if (t.nRanks < 3) { *why = "topo: fewer than three ranks (one receiver pulls everything from the root)"; return false; }
            // with a switch the multicast forms are faster up to a few hundred MiB (measured at 8 GPUs: 16 MiB 65 against
            // 86 us, 256 MiB 584 against 596 us, 1 GiB 2213 against 1996 us)
            if (t.nvls && o.bytes < (384ull << 20)) { *why = "op: below 384 MiB the switch forms are faster"; return false; }
            return true;
        };
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = m.link();                         // every byte enters every receiver once; the root sends it once
            c.ratio = 1.0;
            c.B = m.stageIn ? m.copy() : 0.25 * m.copy();
            c.C = m.lm.launchUs + 8 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    // ---------------- ReduceScatter and AllReduce on ordinary buffers without the stage-in pass: every rank writes block q
    // of its input into rank q's landing copy (stage-in region, two copies taken in turn) and reduces what landed
    {
        auto ordinaryInput = [](const OpDesc& o, const TopoInfo& t, std::string* why) {
            if (o.inRegistered) { *why = "op: the input is registered, the pull form reads it in place"; return false; }
            if (t.nRanks < 2) { *why = "topo: a single rank"; return false; }
            if (o.stageInBytes / 2 < 4096ull * t.nRanks) { *why = "op: the landing zone is too small"; return false; }
            return true;
        };
        AlgEntry e = Base("P2pReduceScatterSoleMeshPush", HCCL_CMD_REDUCE_SCATTER, HCCL_ENGINE_P2P, "MeshPush", DALG_RS_PUSH, AlgoType::MESH);
        e.attrs.dtypeMask = kReduceTypes;
        e.attrs.needsAligned16 = true;
        e.attrs.minBytes = 256ull << 10;
        e.attrs.opCustomCheck = ordinaryInput;
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = 0.25 * m.copy();          // the landed blocks are read once more, locally
            c.C = m.lm.launchUs + m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
        AlgEntry f = Base("P2pAllReduceSoleMeshPushTwoShot", HCCL_CMD_ALLREDUCE, HCCL_ENGINE_P2P, "MeshPushTwoShot", DALG_AR_PUSH_TWOSHOT, AlgoType::TWOSHOT);
        f.attrs.dtypeMask = kReduceTypes;
        f.attrs.needsAligned16 = true;
        f.attrs.minBytes = 256ull << 10;
        f.attrs.opCustomCheck = ordinaryInput;
        f.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            // (push, reduce and pull run one after the other inside a launch and a large message takes several launches:
            // measured 485 GB/s of bus bandwidth at 1 GiB on 8 GPUs, where the staged switch form stays ahead; the
            // staged peer-to-peer two-shot form has the same phases plus the stage-in pass)
            c.A = 2.0 * (m.p - 1) / m.p * m.link();
            c.ratio = 1.0 / m.p;
            c.B = 0.25 * m.copy() + m.copy() / m.p;
            c.C = m.lm.launchUs + 3 * m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(f);
    }
    // ---------------- point to point and barrier
    for (HcclCMDType op : {HCCL_CMD_SEND, HCCL_CMD_RECEIVE, HCCL_CMD_BATCH_SEND_RECV}) {
        const char* name = op == HCCL_CMD_SEND ? "P2pSendSoleMesh" : (op == HCCL_CMD_RECEIVE ? "P2pRecvSoleMesh" : "P2pBatchSendRecvSoleMesh");
        AlgEntry e = Base(name, op, HCCL_ENGINE_P2P, "Mailbox", DALG_P2P_MAILBOX, AlgoType::MESH);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.A = m.link();
            c.B = m.copy();
            c.C = m.lm.launchUs + m.lm.barrierUs;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
    {
        AlgEntry e = Base("P2pBarrierSoleMesh", HCCL_CMD_BARRIER, HCCL_ENGINE_P2P, "Mesh", DALG_BARRIER, AlgoType::MESH);
        e.costCoeff = [](const TopoInfo& t, const OpDesc& o) {
            M m(t, o);
            CostCoeff c;
            c.C = m.lm.launchUs + m.lm.barrierUs;
            c.net = NetType::LOCAL;
            return std::vector<CostCoeff>{c};
        };
        R.Register(e);
    }
}

}  // namespace

void RegisterDeviceAlgorithms()
{
    static bool done = false;
    if (done) return;
    done = true;
    RegisterAll();
}

}  // namespace hccl
