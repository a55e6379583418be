// Thin wrappers over the Blackwell (sm_100a) PTX this library issues by hand:
// mbarrier, TMA tiled loads (cp.async.bulk.tensor, never with cluster
// multicast), tcgen05 tensor-memory allocation, MMA issue, commit, TMEM loads
// and the proxy / tcgen05 fences.  Descriptor layouts follow the PTX ISA
// "tcgen05 matrix descriptors" and "instruction descriptor" tables.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hccl {
namespace sm100 {

__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t TimerNs()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void MbarInit(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(SmemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void MbarInitFence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void MbarExpectTx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(SmemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limitNs`, raises *abortWord and returns false.
// Once the abort word is up every later wait returns false at once.
__device__ __forceinline__ bool MbarWait(uint64_t* bar, uint32_t parity, volatile uint32_t* abortWord, uint64_t limitNs)
{
    if (MbarTryWait(bar, parity)) return true;
    const uint64_t t0 = TimerNs();
    uint32_t spins = 0;
    for (;;) {
        if (MbarTryWait(bar, parity)) return true;
        if ((++spins & 0xFFu) == 0u) {
            if (*abortWord != 0u) return false;
            if (TimerNs() - t0 > limitNs) {
                *abortWord = 1u;
                return false;
            }
        }
    }
}

// ---- TMA -------------------------------------------------------------------
__device__ __forceinline__ void PrefetchTensorMap(const CUtensorMap* m)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tiled load global -> shared, completion on an mbarrier of this CTA.  x is
// the innermost coordinate and must keep x * elementSize a multiple of 16.
__device__ __forceinline__ void TmaLoad2D(void* smemDst, const CUtensorMap* map, uint64_t* bar, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            SmemAddr(smemDst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(SmemAddr(bar)), "r"(x), "r"(y)
        : "memory");
}
// L2 eviction policies for tiled loads: an operand that every wave of tiles re-reads (and that fits the cache) is
// loaded "evict last", the operand that streams through once "evict first", so that the stream does not push the
// reused operand out to HBM.
__device__ __forceinline__ uint64_t L2PolicyEvictLast()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t L2PolicyEvictFirst()
{
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// Untiled bulk copies (both addresses 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void BulkLoadG2S(void* smemDst, const void* gsrc, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(SmemAddr(smemDst)),
                 "l"(gsrc), "r"(bytes), "r"(SmemAddr(bar))
                 : "memory");
}
__device__ __forceinline__ void BulkStoreS2G(void* gdst, const void* smemSrc, uint32_t bytes)
{
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(SmemAddr(smemSrc)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void BulkCommit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Waits until at most `pending` of the most recent bulk groups still read their shared-memory source.
__device__ __forceinline__ void BulkWaitRead(int pending)
{
    switch (pending) {
        case 0: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory"); break;
        case 5: asm volatile("cp.async.bulk.wait_group.read 5;" ::: "memory"); break;
        case 6: asm volatile("cp.async.bulk.wait_group.read 6;" ::: "memory"); break;
        default: asm volatile("cp.async.bulk.wait_group.read 7;" ::: "memory"); break;
    }
}
// Waits until every bulk group of this thread has completed, writes included.
__device__ __forceinline__ void BulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Waits until at most `pending` of the most recent bulk groups are incomplete (their writes not yet performed).
__device__ __forceinline__ void BulkWaitGroup(int pending)
{
    switch (pending) {
        case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
        case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
        case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
        case 3: asm volatile("cp.async.bulk.wait_group 3;" ::: "memory"); break;
        case 4: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;
        default: asm volatile("cp.async.bulk.wait_group 5;" ::: "memory"); break;
    }
}

// Generic-proxy writes (plain stores by other threads / CTAs / GPUs) must be
// made visible to the async proxy (TMA) with this fence, on both sides of the
// flag hand-over.
__device__ __forceinline__ void FenceProxyAsync() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- tcgen05 ---------------------------------------------------------------
__device__ __forceinline__ void TmemAlloc(uint32_t* smemResult, uint32_t nCols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemResult)), "r"(nCols)
                 : "memory");
}
__device__ __forceinline__ void TmemRelinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc(uint32_t taddr, uint32_t nCols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem], bf16/f16 inputs, fp32 accumulate, one CTA.
__device__ __forceinline__ void UmmaF16(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
        "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Makes the mbarrier track completion of all MMAs issued so far by this thread.
__device__ __forceinline__ void UmmaCommit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(SmemAddr(bar)) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives row
// (lane base + i), columns [col, col+32).
__device__ __forceinline__ void TmemLd32x32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void TmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128-byte swizzle (layout type 2), sm_100
// descriptor version 1.  All operand tiles are written by TMA with
// CU_TENSOR_MAP_SWIZZLE_128B and start on a 1024-byte boundary (base offset 0).
//   K-major operand  (rows = M or N, 64 K-elements = 128 B per row):
//     8-row groups 1024 B apart (stride byte offset); leading offset unused (1).
//   MN-major operand (rows = K, 64 MN-elements = 128 B per row, one TMA box per
//     64 MN-elements): 8-row K groups 1024 B apart (stride byte offset), boxes
//     `boxBytes` apart (leading byte offset).
__device__ __forceinline__ uint64_t SmemDescKMajor(uint32_t smemAddr)
{
    return (uint64_t)((smemAddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t SmemDescMnMajor(uint32_t smemAddr, uint32_t boxBytes)
{
    return (uint64_t)((smemAddr & 0x3FFFFu) >> 4) | ((uint64_t)(boxBytes >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// Instruction descriptor for kind::f16: D = fp32, A = B = bf16 (1) or f16 (0).
__host__ __device__ constexpr uint32_t InstrDescF16(int m, int n, bool bf16, bool aMnMajor, bool bMnMajor)
{
    return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((aMnMajor ? 1u : 0u) << 15) | ((bMnMajor ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ bool ElectOne()
{
    uint32_t pred;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "elect.sync _|p, 0xffffffff;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void NamedBarSync(int id, int nThreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nThreads) : "memory"); }

}  // namespace sm100
}  // namespace hccl
