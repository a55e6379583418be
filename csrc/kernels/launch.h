// Host-side launch interface between the operator layer (C++) and the CUDA
// translation units.  Plain C++ header: no device code, usable from g++.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
#include <cstdint>
#include "hccl/hccl_types.h"

namespace hccl {

struct DevComm;
struct CollArgs;
struct P2pArgs;

// Collects the per-rank launches of ranks that share one GPU and issues them as
// ONE cooperative kernel when the last rank has posted (see CollKernelEmu).
class EmuLauncher {
public:
    virtual ~EmuLauncher() = default;
    virtual HcclResult Post(int rank, const void* args, size_t argBytes, int nBlocks, int threads,
                            const void* emuKernel, cudaStream_t stream) = 0;
};

struct LaunchTarget {
    const DevComm* dev;     // host copy of this rank's device communicator
    cudaStream_t stream;
    EmuLauncher* emu;       // non-null: ranks are emulated on one GPU
    int emuRank;
};

// Device algorithms (what the selector chooses among on the GPU engines).
enum DevAlg : int {
    DALG_AR_LL = 0, DALG_AR_ONESHOT, DALG_AR_TWOSHOT, DALG_AR_NVLS,
    DALG_RS_PULL, DALG_RS_NVLS,
    DALG_AG_PULL, DALG_AG_LL,
    DALG_BCAST_ONESHOT, DALG_BCAST_TWOSHOT, DALG_BCAST_NVLS,
    DALG_REDUCE_ONESHOT, DALG_REDUCE_TWOSHOT,
    DALG_SCATTER_PULL, DALG_A2A_PULL, DALG_P2P_MAILBOX, DALG_BARRIER, DALG_TEST_WAIT,
    DALG_RS_LL, DALG_BCAST_LL, DALG_A2A_LL,
    // reductions fused with a cast to another floating type and a scale
    DALG_AR_ONESHOT_CAST, DALG_AR_TWOSHOT_CAST, DALG_RS_CAST,
    // ring and halving-doubling templates
    DALG_RS_RING, DALG_AG_RING, DALG_AR_RHD,
    // switch multicast AllGather, Broadcast as scatter + switch AllGather, AlltoAll through the receivers' slabs
    DALG_AG_NVLS, DALG_BCAST_SCATTER_NVLS, DALG_A2A_PUSH,
    // ordinary buffers without the stage-in pass: blocks pushed into the receivers' slabs
    DALG_RS_PUSH, DALG_AR_PUSH_TWOSHOT,
    // Broadcast of large messages: scatter from the root and AllGather among the others, pipelined piece by piece
    DALG_BCAST_PIPE,
    // AlltoAllV whose size exchange and start barrier run on one block row per rank
    DALG_A2AV_LEADER,
    DALG_COUNT
};

HcclResult LaunchCollective(const LaunchTarget& t, DevAlg alg, HcclDataType dtype, const CollArgs& args, int nBlocks);
// The algorithms of coll_bodies_ext.cuh (outType only matters for the cast forms; pass dtype otherwise).
HcclResult LaunchCollectiveExt(const LaunchTarget& t, DevAlg alg, HcclDataType dtype, HcclDataType outType, const CollArgs& args, int nBlocks);
HcclResult LaunchP2p(const LaunchTarget& t, const P2pArgs& args, int nBlocks);
// Highest number of blocks per emulated rank that still fits one cooperative grid.
int EmuMaxBlocksPerRank(int nRanks);

}  // namespace hccl
