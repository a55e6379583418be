// Symmetric memory: an allocation of the same size on every rank, with every
// rank's copy mapped into every process and (where the box exposes NVLS) a
// multicast alias that addresses all copies at once.
//
// HCCL equivalents: the registered CCL staging buffer whose remote address is
// handed out per channel (ChannelInfo.remoteCclMem, alg_param.h:558-572) and the
// symmetric windows that give the peer VA of user buffers
// (hccl_sym_win_dl.h:28-39).  Three transports, tried in this order:
//   VMM   cuMemCreate + POSIX-fd export/import + cuMemMap (+ cuMulticast*)
//   IPC   cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle (no multicast)
//   LOCAL all ranks on one GPU in one process (emulation): plain cudaMalloc
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>
#include <cuda_runtime.h>
#include "bootstrap.h"
#include "hccl/hccl_types.h"

namespace hccl {

enum class SymTransport : int { NONE = 0, VMM, IPC, LOCAL, USER_IPC };

struct SymSegment {
    size_t size = 0;                 // usable bytes (as requested)
    size_t mappedSize = 0;           // rounded to the mapping granularity
    SymTransport transport = SymTransport::NONE;
    int rank = 0, nRanks = 0;
    void* peer[HCCL_MAX_DEVICE_RANKS] = {nullptr};   // peer[rank] is the local copy
    void* mc = nullptr;              // multicast alias or nullptr
    // bookkeeping for release
    unsigned long long localHandle = 0, mcHandle = 0;
    bool mcBound = false;            // the local allocation is bound to the multicast object
    unsigned long long peerHandle[HCCL_MAX_DEVICE_RANKS] = {0};
    void* ipcBase[HCCL_MAX_DEVICE_RANKS] = {nullptr};   // USER_IPC: what cudaIpcOpenMemHandle returned for each peer
    bool ContainsLocal(const void* p, size_t bytes) const
    {
        const char* b = (const char*)peer[rank];
        return (const char*)p >= b && (const char*)p + bytes <= b + size;
    }
};

// Capabilities of the current device as far as this module is concerned.
struct SymCaps {
    bool vmm = false;       // virtual memory management + POSIX fd handles
    bool multicast = false; // NVLS multicast objects
};
SymCaps QuerySymCaps(int device);

// Collective over `bs`: every rank calls with the same size / wantMulticast.
// `device` must be current.  On failure of the preferred transport all ranks
// agree (over the bootstrap) to fall back to the next one together - the same
// "lowest common capability" rule as the reference's cross-rank engine fallback
// (ccu_fallback.h; op_common.cc:2064-2083).
HcclResult SymAlloc(Bootstrap& bs, int device, size_t size, bool wantMulticast, bool forceIpc, SymSegment* out);
HcclResult SymFree(SymSegment* seg);

// Registration of a buffer the caller allocated itself with cudaMalloc (or a framework allocator on top of it): every
// rank passes its own buffer of `size` bytes; the peers map it through legacy CUDA IPC handles (which work for any
// cudaMalloc allocation, whole allocations only, hence the offset exchange).  Collective.  The segment has no
// multicast alias: operators on it run the peer-to-peer kernels without staging copies.
HcclResult SymRegisterUser(Bootstrap& bs, void* ptr, size_t size, SymSegment* out);

// Emulation: R segments on the current GPU, every "peer" pointer valid locally.
HcclResult SymAllocLocalGroup(int nRanks, size_t size, std::vector<SymSegment>* out);

}  // namespace hccl
