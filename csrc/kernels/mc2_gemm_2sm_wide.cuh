// Wide-tile variant of the two-SM matmul (plain matmul only): a CTA pair works on 256 rows x TWO adjacent column
// tiles at once, one in each of its two TMEM accumulators, so that every k-block of A is loaded once for 512 output
// columns instead of once for 256.
//
// Why: a GPU at its power limit finishes a step when the step's energy has been spent, and with 256 x 256 tiles the
// shared-memory fill traffic from L2 (64 KiB per pair and k-block, about 11 TB/s at full tensor rate) is a large part
// of what a matmul spends beyond the tensor cores.  The wide tile needs 48 KiB per CTA and k-block for twice the
// math (A 16 KiB + two B halves of 16 KiB): a quarter less L2 -> SM traffic per FLOP.  The price: both accumulators
// belong to the tile in flight, so the epilogue no longer overlaps the next tile's main loop; that is a few percent
// of a tile when K is in the thousands and too much when it is not, so the launcher picks this kernel only for
// large K and enough tiles to keep the last wave busy.
//
// Pipeline: four stages of 48 KiB; otherwise the roles, barriers and hand-over of mc2_gemm_2sm.cuh (full[stage] in
// the leader, empty[stage] and tmemFull per CTA through the multicast commit, tmemEmpty in the leader with eight
// arrivals).
#pragma once
#include "mc2_gemm_2sm.cuh"

namespace hccl {
namespace mc2 {

constexpr int kStagesWide = 4;
struct SmemLayoutWide {
    static constexpr int kABytes = kBM * kBK * 2;            // 16 KiB: this CTA's 128 rows of A
    static constexpr int kBBytes = (kBN2 / 2) * kBK * 2;     // 16 KiB: this CTA's half of ONE column tile of B
    static constexpr int kStageBytes = kABytes + 2 * kBBytes;
    static constexpr int kTileBytes = kStagesWide * kStageBytes;   // 192 KiB
    static constexpr int kStagingOff = kTileBytes + 256;
    static constexpr int kTotal = kStagingOff + kEpilogueStagingBytes + 1024;
};

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
    GemmKernel2SmWide(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs g)
{
    using L = SmemLayoutWide;
    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kTileBytes);
    uint64_t* fullBar = bars;                          // [kStagesWide]  (used in the leader)
    uint64_t* emptyBar = bars + kStagesWide;           // [kStagesWide]
    uint64_t* tmemFull = bars + 2 * kStagesWide;       // one: both accumulators complete together
    uint64_t* tmemEmpty = bars + 2 * kStagesWide + 1;  // one (used in the leader)
    uint32_t* tmemBaseSlot = reinterpret_cast<uint32_t*>(bars + 2 * kStagesWide + 2);
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;

    const int warp = threadIdx.x / 32;
    const int cta = (int)blockIdx.x;
    const uint32_t crank = ClusterCtaRank();
    const uint32_t launchEpoch = *reinterpret_cast<volatile uint32_t*>(g.ctl + kCtlEpoch) + 1;

    constexpr uint32_t kTmemCols = 2 * kBN2;
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesWide; ++s) { MbarInit(&fullBar[s], 1); MbarInit(&emptyBar[s], 1); }
        MbarInit(tmemFull, 1);
        MbarInit(tmemEmpty, 2 * (kEpilogueThreads / 32));
        MbarInitFence();
        PrefetchTensorMap(&tmA);
        PrefetchTensorMap(&tmB);
    }
    if (warp == 1) {
        TmemAlloc2(tmemBaseSlot, kTmemCols);
        TmemRelinquish2();
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();
    TcFenceAfter();
    const uint32_t tmemBase = *tmemBaseSlot;
    const int BN = g.bn;
    const int pair = cta >> 1, nPairs = g.nGemmCtas >> 1;
    const int tilesM2 = (g.M + 255) / 256;
    const int tilesNW = (g.tilesN + 1) / 2;             // wide column tiles: (2w, 2w + 1)
    const int nTiles = tilesM2 * tilesNW;
    const int kBlocks = (g.K + kBK - 1) / kBK;
    // grouped raster over (256-row tile, wide column tile): bands of g.rasterGroup (default 8) row tiles, rows fastest
    auto coord = [&](int t, int* mt2, int* ntw) {
        const int kGroup = g.rasterGroup > 0 ? g.rasterGroup : 8;
        const int perBand = kGroup * tilesNW;
        const int band = t / perBand, rem = t % perBand;
        const int first = band * kGroup;
        const int rows = (tilesM2 - first) < kGroup ? (tilesM2 - first) : kGroup;
        *mt2 = first + rem % rows;
        *ntw = rem / rows;
    };

    if (warp == 0) {
        // ===== TMA producer (both CTAs)
        if (ElectOne()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t bHalfBytes = (uint32_t)((BN / 2) * kBK * 2);
            for (int t = pair; t < nTiles && ok; t += nPairs) {
                int mt2, ntw;
                coord(t, &mt2, &ntw);
                const int mt = mt2 * 2 + (int)crank;
                const int nt0 = 2 * ntw;
                const bool second = nt0 + 1 < g.tilesN;
                for (int kb = 0; kb < kBlocks; ++kb) {
                    ok = MbarWait(&emptyBar[stage], phase ^ 1u, abortWord, kWaitLimitNs);
                    if (!ok) break;
                    uint8_t* sa = smem + stage * L::kStageBytes;
                    const uint32_t leaderFull = SmemAddr(&fullBar[stage]) & kPeerBitMask;
                    if (crank == 0) MbarExpectTx(&fullBar[stage], 2u * ((uint32_t)L::kABytes + (second ? 2u : 1u) * bHalfBytes));
                    if (!A_MN) {
                        TmaLoad2D2Sm(sa, &tmA, leaderFull, kb * kBK, mt * kBM);
                    } else {
#pragma unroll
                        for (int j = 0; j < kBM / 64; ++j) TmaLoad2D2Sm(sa + j * (64 * kBK * 2), &tmA, leaderFull, mt * kBM + j * 64, kb * kBK);
                    }
                    for (int h = 0; h < (second ? 2 : 1); ++h) {
                        uint8_t* sb = sa + L::kABytes + h * L::kBBytes;
                        const int nRow = (nt0 + h) * BN + (int)crank * (BN / 2);
                        if (!B_MN) {
                            TmaLoad2D2Sm(sb, &tmB, leaderFull, kb * kBK, nRow);
                        } else {
#pragma unroll
                            for (int j = 0; j < (kBN2 / 2) / 64; ++j)
                                if (j * 64 < BN / 2) TmaLoad2D2Sm(sb + j * (64 * kBK * 2), &tmB, leaderFull, nRow + j * 64, kb * kBK);
                        }
                    }
                    if (++stage == kStagesWide) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                const uint64_t t0 = TimerNs();
                while (TimerNs() - t0 < 200000) {}
            }
        }
    } else if (warp == 1) {
        // ===== MMA issuer: leader CTA only
        if (crank == 0 && ElectOne()) {
            const uint32_t idesc = InstrDescF16(256, BN, true, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t accPhase = 0;
            bool ok = true;
            for (int t = pair; t < nTiles && ok; t += nPairs) {
                int mt2, ntw;
                coord(t, &mt2, &ntw);
                const bool second = 2 * ntw + 1 < g.tilesN;
                ok = MbarWait(tmemEmpty, accPhase ^ 1u, abortWord, kWaitLimitNs);
                if (!ok) break;
                TcFenceAfter();
                for (int kb = 0; kb < kBlocks; ++kb) {
                    ok = MbarWait(&fullBar[stage], phase, abortWord, kWaitLimitNs);
                    if (!ok) break;
                    TcFenceAfter();
                    const uint32_t sa = SmemAddr(smem + stage * L::kStageBytes);
                    const uint64_t da = A_MN ? SmemDescMnMajor(sa, 64 * kBK * 2) : SmemDescKMajor(sa);
                    for (int h = 0; h < (second ? 2 : 1); ++h) {
                        const uint32_t sb = sa + L::kABytes + h * L::kBBytes;
                        const uint64_t db = B_MN ? SmemDescMnMajor(sb, 64 * kBK * 2) : SmemDescKMajor(sb);
                        const uint32_t tmemD = tmemBase + (uint32_t)(h * kBN2);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k) {
                            const uint64_t aStep = (uint64_t)((A_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            const uint64_t bStep = (uint64_t)((B_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            UmmaF16_2Sm(tmemD, da + aStep, db + bStep, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                    }
                    UmmaCommit2Sm(&emptyBar[stage]);
                    if (++stage == kStagesWide) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                UmmaCommit2Sm(tmemFull);
                accPhase ^= 1u;
            }
        }
    } else {
        // ===== epilogue warps 2..5 of both CTAs: each CTA drains its own 128 accumulator rows of both column tiles
        const int quarter = warp & 3;
        const int lane = threadIdx.x & 31;
        uint32_t accPhase = 0;
        bool ok = true;
        for (int t = pair; t < nTiles && ok; t += nPairs) {
            int mt2, ntw;
            coord(t, &mt2, &ntw);
            const int mt = mt2 * 2 + (int)crank;
            ok = MbarWait(tmemFull, accPhase, abortWord, kWaitLimitNs);
            if (!ok) break;
            TcFenceAfter();
            const int row0 = mt * kBM + quarter * 32;
            uint8_t* stg = smem + L::kStagingOff + quarter * kStgWarpBytes;
            for (int h = 0; h < 2; ++h) {
                const int nt = 2 * ntw + h;
                if (nt >= g.tilesN) break;
                const uint32_t taddr = tmemBase + (uint32_t)(h * kBN2) + ((uint32_t)(quarter * 32) << 16);
                const int validCols = g.N - nt * BN;
                DrainTileRows(taddr, BN, stg, lane, validCols, g.M - row0, g.out + (size_t)row0 * g.ldc + (size_t)nt * BN, (size_t)g.ldc);
            }
            TcFenceBefore();
            __syncwarp();
            if (lane == 0) MbarArriveCluster(SmemAddr(tmemEmpty) & kPeerBitMask);
            accPhase ^= 1u;
        }
    }
    TcFenceBefore();
    __syncthreads();
    ClusterSync();
    if (warp == 1) {
        TcFenceAfter();
        TmemDealloc2(tmemBase, kTmemCols);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const uint32_t ticket = atomicAdd(g.ctl + kCtlTicket, 1u);
        if (ticket == gridDim.x - 1) {
            g.ctl[kCtlTicket] = 0;
            *reinterpret_cast<volatile uint32_t*>(g.ctl + kCtlEpoch) = launchEpoch;
            __threadfence();
        }
    }
}

}  // namespace mc2
}  // namespace hccl
