// Launch of one kernel body: a plain launch on this rank's stream, or a post to the group that runs emulated ranks
// as one cooperative kernel.
#pragma once
#include "dev_comm.cuh"
#include "launch.h"
#include "../core/log.h"

namespace hccl {

template <class Body>
HcclResult LaunchBody(const LaunchTarget& t, const typename Body::Args& a, int nBlocks)
{
    if (nBlocks < 1) nBlocks = 1;
    if (nBlocks > kMaxBlocks) nBlocks = kMaxBlocks;
    if (t.emu != nullptr) {
        return t.emu->Post(t.emuRank, &a, sizeof(a), nBlocks, Body::kThreads,
                           reinterpret_cast<const void*>(&CollKernelEmu<Body>), t.stream);
    }
    CollKernel<Body><<<nBlocks, Body::kThreads, 0, t.stream>>>(*t.dev, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        HCCL_ERROR("kernel launch failed: %s", cudaGetErrorString(e));
        return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
