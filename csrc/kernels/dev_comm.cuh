// Device-side view of a communicator and the cross-GPU synchronisation
// primitives every kernel of this library uses.
//
// Role in HCCL terms: this is the counterpart of AivCommBase
// (op_common/algorithm/template/aiv/aiv_communication_base_v2.h): the peer
// buffer table (:223-251), the Record/WaitFlag flag protocol (:475-534) and the
// per-launch tag (:261-278).  Differences that matter on a shared NVSwitch box:
//   * flag values are 64-bit epochs that only grow, so no flag is ever cleared
//     and there is no first-op "clear all flags" barrier;
//   * the epoch lives in device memory, one word per block row, and is advanced
//     by the kernel itself - a captured CUDA graph can be replayed;
//   * every wait is bounded: after `timeoutNs` it records what it was waiting
//     for in a host-visible status block, raises a communicator-wide abort word
//     and returns, and later waits return at once.  No trap, no endless spin.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "dev_types.h"
#include "host_shim.h"

namespace hccl {

__device__ __forceinline__ uint64_t* FlagPtr(const DevComm& c, int ownerRank, int block, int slot, int fromRank)
{
    return reinterpret_cast<uint64_t*>(c.slab[ownerRank] + kSlabFlagsOff) +
           ((size_t)(block * kFlagSlots + slot) * kMaxDevRanks + fromRank) * kFlagStride;
}
__device__ __forceinline__ char* StagePtr(const DevComm& c, int ownerRank) { return c.slab[ownerRank] + kSlabDataOff; }
__device__ __forceinline__ char* StageMcPtr(const DevComm& c) { return c.slabMc ? c.slabMc + kSlabDataOff : nullptr; }

#ifdef HCCL_HOST_SHIM
inline void StReleaseSys(uint64_t* p, uint64_t v) { __atomic_store_n(p, v, __ATOMIC_RELEASE); }
inline uint64_t LdAcquireSys(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_ACQUIRE); }
inline uint64_t LdRelaxedSys(const uint64_t* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
inline uint32_t LdVolatileU32(const uint32_t* p) { return __atomic_load_n(p, __ATOMIC_RELAXED); }
inline uint64_t GlobalTimerNs() { return hostshim::NowNs(); }
#else
__device__ __forceinline__ void StReleaseSys(uint64_t* p, uint64_t v)
{
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t LdAcquireSys(const uint64_t* p)
{
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t LdRelaxedSys(const uint64_t* p)
{
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t LdVolatileU32(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t GlobalTimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#endif

static __device__ __noinline__ void ReportWaitFailure(const DevComm& c, uint32_t kernelId, int block, int slot, int peer,
                                               uint64_t expected, uint64_t seen, uint32_t err)
{
    if (atomicCAS(c.abortWord, 0u, err) == 0u) {
        DevStatus* s = c.status;
        s->kernelId = kernelId;
        s->block = (uint32_t)block;
        s->slot = (uint32_t)slot;
        s->peer = (uint32_t)peer;
        s->rank = (uint32_t)c.rank;
        s->expected = expected;
        s->seen = seen;
        __threadfence_system();
        s->error = err;
        __threadfence_system();
    }
}

// Spin until *flag >= want.  Returns false when the budget ran out or the
// communicator is already aborted.  One thread calls this for one flag.
__device__ __forceinline__ bool WaitFlagGE(const DevComm& c, const uint64_t* flag, uint64_t want, uint32_t kernelId,
                                           int block, int slot, int peer)
{
    uint64_t v = LdAcquireSys(flag);
    if (v >= want) return true;
    if (LdVolatileU32(c.abortWord) != 0u) return false;
    const uint64_t t0 = GlobalTimerNs();
    uint32_t spins = 0;
    for (;;) {
        v = LdAcquireSys(flag);
        if (v >= want) return true;
        HCCL_SPIN_PAUSE();
        if ((++spins & 0x3FFu) == 0u) {
            if (LdVolatileU32(c.abortWord) != 0u) return false;
            if (GlobalTimerNs() - t0 > c.timeoutNs) {
                ReportWaitFailure(c, kernelId, block, slot, peer, want, v, DEV_ERR_TIMEOUT);
                return false;
            }
        }
    }
}

// Epoch handling.  A kernel that performs S cross-rank sync points per block
// reads its row's epoch at entry and publishes epoch+S at exit; sync point k
// (0-based) uses the flag value epoch+k+1.
__device__ __forceinline__ uint64_t LoadEpoch(const DevComm& c, int block)
{
    return *reinterpret_cast<volatile uint64_t*>(c.epochs + block);
}
// Call after the last use of the epoch by every thread of the block.
__device__ __forceinline__ void StoreEpoch(const DevComm& c, int block, uint64_t next)
{
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile uint64_t*>(c.epochs + block) = next;
}

// LL (flag-in-data) ops share ONE counter per communicator: a line's flag has to be unique per op whichever block
// wrote the line last (block rows cover different line ranges from op to op).  Every block reads the counter at
// entry; the last block to finish advances it, which is after all blocks have read it.  Being device-resident it
// survives CUDA-graph replay.
__device__ __forceinline__ uint64_t LoadLLEpoch(const DevComm& c)
{
    return *reinterpret_cast<volatile uint64_t*>(c.epochs + kMaxBlocks);
}
// Credit of the LL forms.  Lines of op `epoch` go into the reader's slot of parity epoch & 1, which op epoch - 2 used
// last.  In the forms where every rank waits for lines of every peer, a rank in op `epoch` knows that all peers have
// entered epoch - 1 and so finished epoch - 2; a one-to-many form (Broadcast: the root waits for nobody, a receiver
// only for the root) gives no such guarantee, and a writer two ops ahead of a slow reader would replace lines the
// reader still polls for.  So every rank tells every peer when it has finished an LL op (flag slot kLLCreditSlot of
// block row 0, value epoch + 1), and before writing the lines of op `epoch` a rank checks that each peer it writes to
// has reported epoch - 2.  In step the check is one read of local memory per peer.
constexpr int kLLCreditSlot = 1;
__device__ __forceinline__ bool LLCreditWait(const DevComm& c, uint64_t epoch, uint32_t kernelId, int block)
{
    HCCL_SHARED(int, s_creditOk);
    if (threadIdx.x == 0) s_creditOk = 1;
    __syncthreads();
    if (epoch >= 2 && (int)threadIdx.x < c.nRanks && (int)threadIdx.x != c.rank) {
        if (!WaitFlagGE(c, FlagPtr(c, c.rank, 0, kLLCreditSlot, threadIdx.x), epoch - 1, kernelId, block, kLLCreditSlot, threadIdx.x)) s_creditOk = 0;
    }
    __syncthreads();
    return s_creditOk != 0;
}
__device__ __forceinline__ void FinishLLEpoch(const DevComm& c, uint64_t epoch, int nBlocks)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        unsigned long long* ticket = reinterpret_cast<unsigned long long*>(c.epochs + kMaxBlocks + 1);
        const unsigned long long t = atomicAdd(ticket, 1ull);
        if (t == (unsigned long long)(nBlocks - 1)) {
            *reinterpret_cast<volatile uint64_t*>(ticket) = 0;
            *reinterpret_cast<volatile uint64_t*>(c.epochs + kMaxBlocks) = epoch + 1;
            __threadfence();
            // every block of this rank has read its lines of this op: the peers may reuse the slots of this parity
            for (int q = 0; q < c.nRanks; ++q)
                if (q != c.rank) StReleaseSys(FlagPtr(c, q, 0, kLLCreditSlot, c.rank), epoch + 1);
        }
    }
}

// The push forms (blocks written into the receivers' stage-in region, no closing barrier) alternate between two
// landing copies.  Which copy an operator uses must not depend on a block row (rows cover different byte ranges from
// operator to operator, and their barrier epochs drift apart when operators use different grids), so the parity comes
// from one counter per communicator that counts push operators: every block reads it at entry, the last block to
// finish advances it.  All ranks issue the same operators in the same order, so the counters agree; being
// device-resident they survive CUDA-graph replay.  Why two copies suffice: a rank that writes for push operator n + 2
// has finished kernel n + 1, in which at least one of its block rows passed a barrier that the peer's row entered
// after the peer's kernel n had ended (stream order).
__device__ __forceinline__ uint64_t LoadPushSeq(const DevComm& c)
{
    return *reinterpret_cast<volatile uint64_t*>(c.epochs + kMaxBlocks + 2);
}
__device__ __forceinline__ void FinishPushSeq(const DevComm& c, uint64_t seq, int nBlocks)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long* ticket = reinterpret_cast<unsigned long long*>(c.epochs + kMaxBlocks + 3);
        const unsigned long long t = atomicAdd(ticket, 1ull);
        if (t == (unsigned long long)(nBlocks - 1)) {
            *reinterpret_cast<volatile uint64_t*>(ticket) = 0;
            *reinterpret_cast<volatile uint64_t*>(c.epochs + kMaxBlocks + 2) = seq + 1;
        }
    }
}

// AlltoAllV with a leader row (A2avLeaderBody) keeps four words per communicator: a count of such operators (read by
// every block at entry, advanced by the last block to finish, like the flag-in-data counter), its ticket, and a
// (tag, largest pair) pair through which block row 0 tells the other rows of ITS rank what the size exchange found.
constexpr int kA2avSeqWord = kMaxBlocks + 4, kA2avTicketWord = kMaxBlocks + 5, kA2avTagWord = kMaxBlocks + 6, kA2avMaxWord = kMaxBlocks + 7;
__device__ __forceinline__ uint64_t LoadA2avSeq(const DevComm& c)
{
    return *reinterpret_cast<volatile uint64_t*>(c.epochs + kA2avSeqWord);
}
__device__ __forceinline__ void FinishA2avSeq(const DevComm& c, uint64_t seq, int nBlocks)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long* ticket = reinterpret_cast<unsigned long long*>(c.epochs + kA2avTicketWord);
        const unsigned long long t = atomicAdd(ticket, 1ull);
        if (t == (unsigned long long)(nBlocks - 1)) {
            *reinterpret_cast<volatile uint64_t*>(ticket) = 0;
            *reinterpret_cast<volatile uint64_t*>(c.epochs + kA2avSeqWord) = seq + 1;
        }
    }
}

// Barrier among the blocks with index `block` of all ranks, on flag slot `slot`.
// Everything the calling block wrote before the barrier (local or peer memory)
// is visible to every participating block after it.  All threads of the block
// must call it.  Returns false on timeout / abort (data is then meaningless but
// the kernel can run to its end without waiting again).
__device__ __forceinline__ bool RankBarrier(const DevComm& c, int block, int slot, uint64_t value, uint32_t kernelId)
{
    HCCL_SHARED(int, s_ok);
    __syncthreads();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < c.nRanks) {
        const int peer = threadIdx.x;
        // the release store at system scope orders everything the block wrote before the __syncthreads above (release
        // is cumulative over what the storing thread has observed), so no separate fence is needed
        StReleaseSys(FlagPtr(c, peer, block, slot, c.rank), value);
        if (!WaitFlagGE(c, FlagPtr(c, c.rank, block, slot, peer), value, kernelId, block, slot, peer)) s_ok = 0;
    }
    __syncthreads();
    return s_ok != 0;
}

// One-directional signal / wait pair (producer -> consumer), same visibility
// guarantees as the barrier.  Call SignalPeer from ONE thread after a
// __syncthreads() that follows the data writes.
__device__ __forceinline__ void SignalPeer(const DevComm& c, int peer, int block, int slot, uint64_t value)
{
    __threadfence_system();
    StReleaseSys(FlagPtr(c, peer, block, slot, c.rank), value);
}
__device__ __forceinline__ bool WaitPeer(const DevComm& c, int peer, int block, int slot, uint64_t value,
                                         uint32_t kernelId)
{
    return WaitFlagGE(c, FlagPtr(c, c.rank, block, slot, peer), value, kernelId, block, slot, peer);
}

// Stuck-detection counters (reference: stuck_detect_counter_helper.h; AIV
// EmitStuckCounter aiv_communication_base_v2.h:368-378).  Block 0 bumps `head`
// at entry and `tail` at exit; a host watchdog compares them.
// The running values live in device memory (no read crosses PCIe); each bump is
// mirrored to the host-mapped status block with one posted write.
__device__ __forceinline__ void OpHead(const DevComm& c, int block)
{
    if (block == 0 && threadIdx.x == 0) {
        volatile uint64_t* h = c.epochs + 2 * kMaxBlocks;
        const uint64_t v = *h + 1;
        *h = v;
        c.status->head = v;
    }
}
__device__ __forceinline__ void OpTail(const DevComm& c, int block)
{
    if (block == 0 && threadIdx.x == 0) {
        volatile uint64_t* t = c.epochs + 2 * kMaxBlocks + 1;
        const uint64_t v = *t + 1;
        *t = v;
        c.status->tail = v;
    }
}

// Kernel entry wrappers: `Body` is a struct with `using Args = ...` and
// `static __device__ void Run(const DevComm&, const Args&, int block, int nBlocks)`.
// The `Emu` form runs R ranks inside one cooperative grid (rank = blockIdx / nb),
// used when fewer GPUs than ranks are available: blocks of different ranks wait
// on one another, so they must be co-resident, which only a single cooperative
// launch guarantees.
#ifndef HCCL_HOST_SHIM
template <class Body>
__global__ void __launch_bounds__(Body::kThreads) CollKernel(DevComm c, typename Body::Args a)
{
    Body::Run(c, a, (int)blockIdx.x, (int)gridDim.x);
}
template <class Body>
__global__ void __launch_bounds__(Body::kThreads)
    CollKernelEmu(const DevComm* cs, const typename Body::Args* as, int blocksPerRank)
{
    const int r = (int)blockIdx.x / blocksPerRank;
    Body::Run(cs[r], as[r], (int)blockIdx.x % blocksPerRank, blocksPerRank);
}
#endif

}  // namespace hccl
