#include "auto_selector.h"
#include <algorithm>

namespace hccl {
namespace {

constexpr uint64_t KiB = 1024, MiB = 1024 * 1024;
bool Pow2(uint32_t p) { return p && !(p & (p - 1)); }

// ---------------------------------------------------------------- host engine (the reference's cut points)
std::string HostTree(const ThresholdInput& in)
{
    const bool multi = in.levels > 1;
    const char* logAlg = Pow2(in.nRanks) ? "RHD" : "NHR";
    switch (in.op) {
        case HCCL_CMD_ALLREDUCE:
            if (in.strictOrder) return "HostAllReduceStrictOrderedMesh";
            if (multi) return in.levels > 2 ? "HostAllReduceSequenceMeshNHRNHR" : (in.bytes >= 32 * MiB ? "HostAllReduceParallelMeshNHR" : "HostAllReduceSequenceMeshNHR");
            if (in.bytes <= 16 * KiB && in.nRanks <= 8) return "HostAllReduceSoleMeshOneShot";
            if (in.bytes <= 512 * KiB && in.nRanks <= 8) return "HostAllReduceSoleMeshTwoShot";
            if (in.bytes >= 32 * MiB) return "HostAllReduceSoleRing";
            return std::string("HostAllReduceSole") + logAlg;
        case HCCL_CMD_REDUCE_SCATTER:
            if (in.strictOrder) return "HostReduceScatterStrictOrderedMesh";
            if (multi) return "HostReduceScatterSequenceMeshNHR";
            if (in.bytes <= 512 * KiB && in.nRanks <= 8) return "HostReduceScatterSoleMesh";
            return std::string("HostReduceScatterSole") + logAlg;
        case HCCL_CMD_ALLGATHER:
            if (multi) return "HostAllGatherSequenceMeshNHR";
            if (in.bytes <= 512 * KiB && in.nRanks <= 8) return "HostAllGatherSoleMesh";
            return std::string("HostAllGatherSole") + logAlg;
        case HCCL_CMD_BROADCAST:
            if (multi) return "HostBroadcastSequenceMeshNHR";
            if (in.bytes <= 16 * KiB) return "HostBroadcastSoleMeshOneShot";
            return in.nRanks <= 8 ? "HostBroadcastSoleMeshTwoShot" : "HostBroadcastSoleNHR";
        case HCCL_CMD_REDUCE:
            if (multi) return "HostReduceSequenceMeshNHR";
            if (in.bytes <= 16 * KiB) return "HostReduceSoleMeshOneShot";
            return in.nRanks <= 8 ? "HostReduceSoleMeshTwoShot" : "HostReduceSoleNHR";
        case HCCL_CMD_SCATTER:
            if (multi) return "HostScatterSequenceMeshMesh";
            return in.nRanks > 8 ? "HostScatterSoleNB" : "HostScatterSoleMesh";
        case HCCL_CMD_ALLTOALL: case HCCL_CMD_ALLTOALLV: case HCCL_CMD_ALLTOALLVC: {
            const std::string base = in.op == HCCL_CMD_ALLTOALL ? "HostAlltoAll" : in.op == HCCL_CMD_ALLTOALLV ? "HostAlltoAllV" : "HostAlltoAllVC";
            if (multi) return base + "HierMeshMesh";
            // pairwise avoids incast once the per-pair block is large (Pairwise.md) and needs full boards of 8
            return base + (in.nRanks % 16 == 0 && in.bytes / std::max<uint32_t>(1, in.nRanks) >= 1 * MiB ? "SolePairwise" : "SoleMesh");
        }
        case HCCL_CMD_BARRIER:
            if (multi) return "HostBarrierSequenceMeshNHR";
            return in.nRanks <= 8 ? "HostBarrierSoleMesh" : (Pow2(in.nRanks) ? "HostBarrierSoleRHD" : "HostBarrierSoleNHR");
        default: return "";
    }
}

// ---------------------------------------------------------------- device engines (measured cross-over points, 8 GPUs)
std::string DeviceTree(const ThresholdInput& in)
{
    switch (in.op) {
        case HCCL_CMD_ALLREDUCE:
            if (in.bytes <= 64 * KiB) return "P2pAllReduceSoleMeshLL";
            if (in.bytes <= 512 * KiB) return "P2pAllReduceSoleMeshOneShot";
            return in.nvls && !in.strictOrder ? "NvlsAllReduceSoleMesh" : "P2pAllReduceSoleMeshTwoShot";
        case HCCL_CMD_REDUCE_SCATTER:
            if (in.bytes <= 1 * MiB) return "P2pReduceScatterSoleMeshLL";
            return in.nvls && !in.strictOrder ? "NvlsReduceScatterSoleMesh" : "P2pReduceScatterSoleMesh";
        case HCCL_CMD_REDUCE_SCATTER_V:
            return in.nvls && !in.strictOrder ? "NvlsReduceScatterVSoleMesh" : "P2pReduceScatterVSoleMesh";
        case HCCL_CMD_ALLGATHER:
            return in.bytes <= 2 * MiB ? "P2pAllGatherSoleMeshLL" : "P2pAllGatherSoleMesh";
        case HCCL_CMD_ALLGATHER_V: return "P2pAllGatherVSoleMesh";
        case HCCL_CMD_BROADCAST:
            if (in.bytes <= 64 * KiB) return "P2pBroadcastSoleMeshLL";
            if (in.bytes <= 2 * MiB) return "P2pBroadcastSoleMeshOneShot";
            return in.nvls ? "NvlsBroadcastSoleMesh" : "P2pBroadcastSoleMeshTwoShot";
        case HCCL_CMD_REDUCE:
            return in.bytes <= 512 * KiB ? "P2pReduceSoleMeshOneShot" : "P2pReduceSoleMeshTwoShot";
        case HCCL_CMD_SCATTER: return "P2pScatterSoleMesh";
        case HCCL_CMD_ALLTOALL: return in.bytes <= 2 * MiB ? "P2pAlltoAllSoleMeshLL" : "P2pAlltoAllSoleMesh";
        case HCCL_CMD_ALLTOALLV: return "P2pAlltoAllVSoleMesh";
        case HCCL_CMD_ALLTOALLVC: return "P2pAlltoAllVCSoleMesh";
        case HCCL_CMD_SEND: return "P2pSendSoleMesh";
        case HCCL_CMD_RECEIVE: return "P2pRecvSoleMesh";
        case HCCL_CMD_BATCH_SEND_RECV: return "P2pBatchSendRecvSoleMesh";
        case HCCL_CMD_BARRIER: return "P2pBarrierSoleMesh";
        default: return "";
    }
}

}  // namespace

std::string ThresholdSelect(const ThresholdInput& in) { return in.hostEngine ? HostTree(in) : DeviceTree(in); }

ThresholdInput ThresholdInputOf(const TopoInfo& topo, const OpDesc& op)
{
    ThresholdInput in;
    in.op = op.op;
    in.bytes = op.bytes;
    in.nRanks = topo.nRanks;
    in.levels = topo.nPods > 1 ? 3 : (topo.nServers > 1 ? 2 : 1);
    in.hostEngine = topo.level0Link == LinkKind::HOST_MEM && topo.deviceName.empty();
    const bool reduces = op.op == HCCL_CMD_ALLREDUCE || op.op == HCCL_CMD_REDUCE_SCATTER || op.op == HCCL_CMD_REDUCE_SCATTER_V;
    in.nvls = topo.nvls && (reduces ? op.inMulticast : op.outMulticast);
    in.strictOrder = op.det == Deterministic::STRICT;
    return in;
}

}  // namespace hccl
