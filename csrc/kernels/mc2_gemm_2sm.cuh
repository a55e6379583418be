// Two-SM variant of the MC2 matmul pipeline: a cluster of two CTAs works on one
// 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
// Each CTA of the pair loads its own 128 rows of A and its own 128 of the 256
// B rows (N split), so a k-block costs 32 KiB of shared memory per CTA instead
// of 48 KiB: a third less L2 -> SM traffic per FLOP and six pipeline stages in
// the same shared memory.  The leader CTA (cluster rank 0) issues the MMAs;
// they read both CTAs' shared memory and write 128 accumulator rows into each
// CTA's TMEM.  Hand-over:
//   full[stage]    lives in the leader; BOTH producers' TMA loads complete on
//                  it (cp.async.bulk.tensor ... cta_group::2 with the barrier
//                  address of cluster rank 0; no multicast anywhere)
//   empty[stage]   one per CTA; tcgen05.commit.cta_group::2 with the commit
//                  multicast mask 0b11 arrives on both
//   tmemFull[acc]  one per CTA, same multicast commit
//   tmemEmpty[acc] lives in the leader, 8 arrivals: the four epilogue warps of
//                  each CTA (the follower arrives through the cluster window)
// Epilogues, tile orders, worker CTAs and flag protocols are those of the
// one-SM kernel (mc2_gemm.cuh); a CTA of the pair simply owns its 128-row half.
#pragma once
#include "mc2_gemm.cuh"

namespace hccl {
namespace mc2 {

constexpr int kStages2 = 6;
constexpr int kBN2 = 256;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;     // clears the cluster-rank bit of a shared::cluster address: rank 0's copy

struct SmemLayout2 {
    static constexpr int kABytes = kBM * kBK * 2;            // 16 KiB: this CTA's 128 rows of A
    static constexpr int kBBytes = (kBN2 / 2) * kBK * 2;     // 16 KiB: this CTA's 128 of the 256 B rows
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTileBytes = kStages2 * kStageBytes;   // 192 KiB
    static constexpr int kStagingOff = kTileBytes + 256;
    static constexpr int kTotal = kStagingOff + kEpilogueStagingBytes + 1024;
};

__device__ __forceinline__ uint32_t ClusterCtaRank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void ClusterSync()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void TmaLoad2D2Sm(void* smemDst, const CUtensorMap* map, uint32_t leaderBarAddr, int x, int y)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            SmemAddr(smemDst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(leaderBarAddr), "r"(x), "r"(y)
        : "memory");
}
// The same load with an L2 eviction policy (see L2PolicyEvictLast / L2PolicyEvictFirst).
__device__ __forceinline__ void TmaLoad2D2SmHint(void* smemDst, const CUtensorMap* map, uint32_t leaderBarAddr, int x, int y, uint64_t policy)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(
            SmemAddr(smemDst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(leaderBarAddr), "r"(x), "r"(y), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void UmmaF16_2Sm(uint32_t tmemD, uint64_t descA, uint64_t descB, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmemD),
        "l"(descA), "l"(descB), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the barrier at the same offset in both CTAs once all MMAs issued so far have completed.
__device__ __forceinline__ void UmmaCommit2Sm(uint64_t* bar)
{
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(SmemAddr(bar)),
                 "h"(mask)
                 : "memory");
}
__device__ __forceinline__ void MbarArriveCluster(uint32_t clusterAddr)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(clusterAddr) : "memory");
}
__device__ __forceinline__ void TmemAlloc2(uint32_t* smemResult, uint32_t nCols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(smemResult)), "r"(nCols) : "memory");
}
__device__ __forceinline__ void TmemRelinquish2() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemDealloc2(uint32_t taddr, uint32_t nCols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(nCols) : "memory");
}

// Pair tile index -> (256-row tile, 256-column tile), same orders as TileCoord but in units of 256 rows.
template <int MODE>
__device__ __forceinline__ void TileCoord2(const GemmArgs& g, int t, int tilesM2, int* mt2, int* nt)
{
    if (MODE == MODE_AG) {
        // shards in the order rank, rank + 1, ...; inside a shard bands of row tiles walked column by column (see TileCoord)
        const int rowTiles = g.mPerRank / 256;
        const int tilesPerRank = rowTiles * g.tilesN;
        const int step = t / tilesPerRank, rem = t % tilesPerRank;
        const int src = (g.rank + step) % g.nRanks;
        const int band = rowTiles < kAgBandRows ? rowTiles : kAgBandRows;
        const int perBand = band * g.tilesN;
        const int first = (rem / perBand) * band, r2 = rem % perBand;
        const int rows = (rowTiles - first) < band ? (rowTiles - first) : band;
        *mt2 = src * rowTiles + first + r2 % rows;
        *nt = r2 / rows;
    } else if (MODE == MODE_RS) {
        const int rowTiles = g.mPerRank / 256;
        const int n = t / tilesM2, rem = t % tilesM2;
        const int step = rem / rowTiles;
        const int dstRank = (g.rank + 1 + step) % g.nRanks;
        *mt2 = dstRank * rowTiles + rem % rowTiles;
        *nt = n;
    } else {
        // grouped raster: bands of 8 row tiles, walked column by column, so that the ~74 tiles in flight touch about
        // 8 row tiles of A and 9 column tiles of B instead of all of A
        const int kGroup = g.rasterGroup > 0 ? g.rasterGroup : 8;
        const int perBand = kGroup * g.tilesN;
        const int band = t / perBand, rem = t % perBand;
        const int first = band * kGroup;
        const int rows = (tilesM2 - first) < kGroup ? (tilesM2 - first) : kGroup;
        *mt2 = first + rem % rows;
        *nt = rem / rows;
    }
}

template <bool A_MN, bool B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    GemmKernel2Sm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmAOwn,
                  const GemmArgs g, const DevComm c)
{
    using L = SmemLayout2;
    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kTileBytes);
    uint64_t* fullBar = bars;                       // [kStages2]  (used in the leader)
    uint64_t* emptyBar = bars + kStages2;           // [kStages2]
    uint64_t* tmemFull = bars + 2 * kStages2;       // [2]
    uint64_t* tmemEmpty = bars + 2 * kStages2 + 2;  // [2]       (used in the leader)
    uint32_t* tmemBaseSlot = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 4);
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;

    const int warp = threadIdx.x / 32;
    const int cta = (int)blockIdx.x;
    const uint32_t crank = ClusterCtaRank();
    const uint32_t launchEpoch = *reinterpret_cast<volatile uint32_t*>(g.ctl + kCtlEpoch) + 1;

    if (cta >= g.nGemmCtas) {
        const int worker = cta - g.nGemmCtas, nWorkers = (int)gridDim.x - g.nGemmCtas;
        if (MODE == MODE_AG) {
            if (g.agPush) GatherPushWorker(c, g, worker, nWorkers);
            else GatherWorker(c, g, worker, nWorkers, smem, bars);
        }
        if (MODE == MODE_RS) ReduceWorker<kBN2>(c, g, worker, nWorkers, (uint64_t)launchEpoch);   // fused modes keep 256-wide tiles
    } else {
        constexpr uint32_t kTmemCols = 2 * kBN2;
        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages2; ++s) { MbarInit(&fullBar[s], 1); MbarInit(&emptyBar[s], 1); }
            for (int a = 0; a < 2; ++a) { MbarInit(&tmemFull[a], 1); MbarInit(&tmemEmpty[a], 2 * (kEpilogueThreads / 32)); }
            MbarInitFence();
            PrefetchTensorMap(&tmA);
            PrefetchTensorMap(&tmB);
            if (MODE == MODE_AG) PrefetchTensorMap(&tmAOwn);
        }
        if (warp == 1) {
            TmemAlloc2(tmemBaseSlot, kTmemCols);
            TmemRelinquish2();
        }
        TcFenceBefore();
        __syncthreads();
        ClusterSync();               // the peer's barriers exist before anything arrives on them
        TcFenceAfter();
        const uint32_t tmemBase = *tmemBaseSlot;
        const int BN = g.bn;                        // column tile width of this launch (accumulators stay 256 columns apart)
        const int pair = cta >> 1, nPairs = g.nGemmCtas >> 1;
        const int tilesM2 = (g.M + 255) / 256;
        const int nTiles = tilesM2 * g.tilesN;
        const int kBlocks = (g.K + kBK - 1) / kBK;

        if (warp == 0) {
            // ===== TMA producer (both CTAs): own 128 rows of A, own 128 rows of B, completion on the LEADER's full barrier
            if (ElectOne()) {
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                MC2_TR(long long trReady = 0, trEmpty = 0; const long long trC0 = clock64(); uint64_t trFirst = 0; int trTiles = 0; if (g.trace) g.trace[(size_t)cta * kTraceWords + TR_START_NS] = TimerNs();)
                const uint64_t polA = g.l2HintA == 1 ? L2PolicyEvictLast() : L2PolicyEvictFirst();
                const uint64_t polB = g.l2HintB == 1 ? L2PolicyEvictLast() : L2PolicyEvictFirst();
                for (int t = pair; t < nTiles && ok; t += nPairs) {
                    int mt2, nt;
                    TileCoord2<MODE>(g, t, tilesM2, &mt2, &nt);
                    const int mt = mt2 * 2 + (int)crank;           // this CTA's 128-row tile
                    const int ownFirst = g.rank * (g.mPerRank / kBM);
                    const bool own = MODE == MODE_AG && mt >= ownFirst && mt < ownFirst + g.mPerRank / kBM;
                    const CUtensorMap* mapA = own ? &tmAOwn : &tmA;     // own rows: read from the shard itself, no wait
                    const int rowA = (own ? mt - ownFirst : mt) * kBM;
                    if (MODE == MODE_AG && !own) {
                        const int nWorkers = (int)gridDim.x - g.nGemmCtas;
                        MC2_TR(const long long c0 = clock64();)
                        if (g.agPush) ok = SpinUntilGE64(g.agReady[g.rank] + mt, (uint64_t)g.K * 2 * kBM, abortWord);
                        else ok = SpinUntilGE(g.ctl + kCtlReady + mt, (uint32_t)nWorkers, abortWord);
                        MC2_TR(trReady += clock64() - c0; if (trFirst == 0) trFirst = TimerNs();)
                        FenceProxyAsync();
                        if (!ok) break;
                    }
                    MC2_TR(++trTiles;)
                    for (int kb = 0; kb < kBlocks; ++kb) {
                        MC2_TR(const long long c1 = clock64();)
                        ok = MbarWait(&emptyBar[stage], phase ^ 1u, abortWord, kWaitLimitNs);
                        MC2_TR(trEmpty += clock64() - c1;)
                        if (!ok) break;
                        uint8_t* sa = smem + stage * L::kStageBytes;
                        uint8_t* sb = sa + L::kABytes;
                        const uint32_t leaderFull = SmemAddr(&fullBar[stage]) & kPeerBitMask;
                        if (crank == 0) MbarExpectTx(&fullBar[stage], (uint32_t)(2 * (L::kABytes + (BN / 2) * kBK * 2)));
                        if (!A_MN) {
                            if (g.l2HintA != 0) TmaLoad2D2SmHint(sa, mapA, leaderFull, kb * kBK, rowA, polA);
                            else TmaLoad2D2Sm(sa, mapA, leaderFull, kb * kBK, rowA);
                        } else {
#pragma unroll
                            for (int j = 0; j < kBM / 64; ++j) {
                                if (g.l2HintA != 0) TmaLoad2D2SmHint(sa + j * (64 * kBK * 2), &tmA, leaderFull, mt * kBM + j * 64, kb * kBK, polA);
                                else TmaLoad2D2Sm(sa + j * (64 * kBK * 2), &tmA, leaderFull, mt * kBM + j * 64, kb * kBK);
                            }
                        }
                        const int nRow = nt * BN + (int)crank * (BN / 2);
                        if (!B_MN) {
                            if (g.l2HintB != 0) TmaLoad2D2SmHint(sb, &tmB, leaderFull, kb * kBK, nRow, polB);
                            else TmaLoad2D2Sm(sb, &tmB, leaderFull, kb * kBK, nRow);
                        } else {
#pragma unroll
                            for (int j = 0; j < (kBN2 / 2) / 64; ++j) {
                                if (j * 64 >= BN / 2) continue;
                                if (g.l2HintB != 0) TmaLoad2D2SmHint(sb + j * (64 * kBK * 2), &tmB, leaderFull, nRow + j * 64, kb * kBK, polB);
                                else TmaLoad2D2Sm(sb + j * (64 * kBK * 2), &tmB, leaderFull, nRow + j * 64, kb * kBK);
                            }
                        }
                        if (++stage == kStages2) { stage = 0; phase ^= 1u; }
                    }
                }
                if (!ok) {
                    const uint64_t t0 = TimerNs();
                    while (TimerNs() - t0 < 200000) {}
                }
                MC2_TR(if (g.trace) {
                    uint64_t* w = g.trace + (size_t)cta * kTraceWords;
                    w[TR_PROD_READY_CLK] = (uint64_t)trReady; w[TR_PROD_FIRST_REMOTE_NS] = trFirst; w[TR_PROD_EMPTY_CLK] = (uint64_t)trEmpty;
                    w[TR_PROD_END_NS] = TimerNs(); w[TR_TILES] = (uint64_t)trTiles; w[TR_EPI_PIECES] = (uint64_t)(clock64() - trC0);   // producer's cycles: the clock rate
                })
            }
        } else if (warp == 1) {
            // ===== MMA issuer: leader CTA only
            if (crank == 0 && ElectOne()) {
                const uint32_t idesc = InstrDescF16(256, BN, true, A_MN, B_MN);
                int stage = 0;
                uint32_t phase = 0;
                int acc = 0;
                uint32_t accPhase = 0;
                bool ok = true;
                MC2_TR(long long trFull = 0, trTmem = 0;)
                for (int t = pair; t < nTiles && ok; t += nPairs) {
                    MC2_TR(const long long c0 = clock64();)
                    ok = MbarWait(&tmemEmpty[acc], accPhase ^ 1u, abortWord, kWaitLimitNs);
                    MC2_TR(trTmem += clock64() - c0;)
                    if (!ok) break;
                    TcFenceAfter();
                    const uint32_t tmemD = tmemBase + (uint32_t)(acc * kBN2);
                    for (int kb = 0; kb < kBlocks; ++kb) {
                        MC2_TR(const long long c1 = clock64();)
                        ok = MbarWait(&fullBar[stage], phase, abortWord, kWaitLimitNs);
                        MC2_TR(trFull += clock64() - c1;)
                        if (!ok) break;
                        TcFenceAfter();
                        const uint32_t sa = SmemAddr(smem + stage * L::kStageBytes);
                        const uint32_t sb = sa + L::kABytes;
                        const uint64_t da = A_MN ? SmemDescMnMajor(sa, 64 * kBK * 2) : SmemDescKMajor(sa);
                        const uint64_t db = B_MN ? SmemDescMnMajor(sb, 64 * kBK * 2) : SmemDescKMajor(sb);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k) {
                            const uint64_t aStep = (uint64_t)((A_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            const uint64_t bStep = (uint64_t)((B_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            UmmaF16_2Sm(tmemD, da + aStep, db + bStep, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                        UmmaCommit2Sm(&emptyBar[stage]);
                        if (++stage == kStages2) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    UmmaCommit2Sm(&tmemFull[acc]);
                    if (++acc == 2) { acc = 0; accPhase ^= 1u; }
                }
                MC2_TR(if (g.trace) {
                    uint64_t* w = g.trace + (size_t)cta * kTraceWords;
                    w[TR_MMA_FULL_CLK] = (uint64_t)trFull; w[TR_MMA_TMEM_CLK] = (uint64_t)trTmem; w[TR_MMA_END_NS] = TimerNs();
                })
            }
        } else {
            // ===== epilogue warps 2..5 of both CTAs: each CTA drains its own 128 accumulator rows
            const int quarter = warp & 3;
            const int lane = threadIdx.x & 31;
            int acc = 0;
            uint32_t accPhase = 0;
            bool ok = true;
            const size_t parityOff = (launchEpoch & 1u) * g.xchgParityElems;
            bool pushLeft = MODE == MODE_AG && g.agPush == kAgPushCoop;
            bool reduceLeft = MODE == MODE_RS && (warp - 2) < g.rsCoop;      // g.rsCoop of the four epilogue warps reduce
            int reducePending = -1;
            MC2_TR(long long trPush = 0, trDrain = 0, trWait = 0, trTail = 0; const bool trMe = g.trace != nullptr && warp == 3 && lane == 0;)
            if (pushLeft && cta == 0 && warp == 2) {
                CoopPushOpen(c, g, launchEpoch, lane);
                MC2_TR(if (g.trace && lane == 0) g.trace[TR_GO_NS] = TimerNs();)
            }
            for (int t = pair; t < nTiles && ok; t += nPairs) {
                int mt2, nt;
                TileCoord2<MODE>(g, t, tilesM2, &mt2, &nt);
                const int mt = mt2 * 2 + (int)crank;
                MC2_TR(const long long c0 = clock64();)
                if (MODE == MODE_AG && pushLeft) pushLeft = CoopPushWhileWaiting(g, launchEpoch, lane, &tmemFull[acc], accPhase);
                if (MODE == MODE_RS && reduceLeft) reduceLeft = CoopReduceWhileWaiting(g, launchEpoch, lane, &reducePending, &tmemFull[acc], accPhase);
                MC2_TR(const long long c1 = clock64(); trPush += c1 - c0;)
                ok = MbarWait(&tmemFull[acc], accPhase, abortWord, kWaitLimitNs);
                MC2_TR(const long long c2 = clock64(); trWait += c2 - c1;)
                if (!ok) break;
                TcFenceAfter();
                const int row0 = mt * kBM + quarter * 32;
                const uint32_t taddr = tmemBase + (uint32_t)(acc * kBN2) + ((uint32_t)(quarter * 32) << 16);
                uint8_t* stg = smem + L::kStagingOff + quarter * kStgWarpBytes;
                const int validCols = g.N - nt * BN;
                // a warp's 32 rows lie in one rank's row block (blocks are multiples of 128 rows) and `stride` apart
                const int validRows = g.M - row0;
                if (MODE == MODE_RS) {
                    const int dst = row0 / g.mPerRank;
                    __nv_bfloat16* base = nullptr;
                    if (row0 < g.M && dst < g.nRanks) {
                        if (g.xchgMc != nullptr) base = g.xchg[g.rank] + parityOff + (size_t)row0 * g.N + (size_t)nt * BN;
                        else base = g.xchg[dst] + parityOff + (size_t)g.rank * g.mPerRank * g.N + (size_t)(row0 - dst * g.mPerRank) * g.N + (size_t)nt * BN;
                    }
                    DrainTileRows(taddr, BN, stg, lane, validCols, base != nullptr ? validRows : 0, base, (size_t)g.N);
                } else {
                    __nv_bfloat16* base = g.out + (size_t)row0 * g.ldc + (size_t)nt * BN;
                    DrainTileRows(taddr, BN, stg, lane, validCols, validRows, base, (size_t)g.ldc);
                }
                TcFenceBefore();
                __syncwarp();
                MC2_TR(trDrain += clock64() - c2;)
                if (lane == 0) MbarArriveCluster(SmemAddr(&tmemEmpty[acc]) & kPeerBitMask);     // the leader's barrier
                if (++acc == 2) { acc = 0; accPhase ^= 1u; }
                if (MODE == MODE_RS) {
                    // the barrier orders all epilogue threads' stores before the publishing thread, whose fence (cumulative)
                    // then covers them: one system fence per tile instead of one per thread
                    NamedBarSync(1, kEpilogueThreads);
                    if (threadIdx.x == 64 && mt * kBM < g.M) {
                        const int dst = (mt * kBM) / g.mPerRank;
                        const int tileId = (mt % (g.mPerRank / kBM)) * g.tilesN + nt;
                        __threadfence_system();
                        StReleaseSys(g.tileFlag[dst] + (size_t)g.rank * g.maxTiles + tileId, (uint64_t)launchEpoch);
                    }
                }
            }
            MC2_TR(const long long c3 = clock64();)
            if (MODE == MODE_AG && pushLeft) CoopPushDrain(g, launchEpoch, lane);
            if (MODE == MODE_RS && reduceLeft) CoopReduceDrain(g, launchEpoch, lane, &reducePending);
            MC2_TR(trTail = clock64() - c3;
                   if (trMe) {
                       uint64_t* w = g.trace + (size_t)cta * kTraceWords;
                       w[TR_EPI_PUSH_CLK] = (uint64_t)trPush; w[TR_EPI_DRAIN_CLK] = (uint64_t)trDrain; w[TR_EPI_FULL_CLK] = (uint64_t)trWait;
                       w[TR_EPI_TAIL_PUSH_CLK] = (uint64_t)trTail; w[TR_EPI_END_NS] = TimerNs();
                   })
        }
        // teardown: nobody leaves while its peer may still touch its shared memory, barriers or TMEM
        TcFenceBefore();
        __syncthreads();
        ClusterSync();
        if (warp == 1) {
            TcFenceAfter();
            TmemDealloc2(tmemBase, kTmemCols);
        }
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t ticket = atomicAdd(g.ctl + kCtlTicket, 1u);
        if (ticket == gridDim.x - 1) {
            if (MODE == MODE_AG) {
                const int n = g.nRanks * (g.mPerRank / kBM);
                for (int i = 0; i < n; ++i) g.ctl[kCtlReady + i] = 0;
                if (g.agPush)
                    for (int i = 0; i < n; ++i) g.agReady[g.rank][i] = 0;      // peers write again only after the next start barrier
            }
            g.ctl[kCtlTicket] = 0;
            g.ctl[kCtlPushNext] = 0;
            g.ctl[kCtlReduceNext] = 0;
            *reinterpret_cast<volatile uint32_t*>(g.ctl + kCtlEpoch) = launchEpoch;
            __threadfence();
        }
    }
}

}  // namespace mc2
}  // namespace hccl
