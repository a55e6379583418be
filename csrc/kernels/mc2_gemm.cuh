// tcgen05 / TMEM GEMM pipeline shared by the MC2 (matmul + collective) kernels.
//
// HCCL ships only the resource half of MC2 (hccl_mc2.h; the isMc2 hooks in
// alg_param.h:784); the fused AllGather->Matmul, Matmul->ReduceScatter and
// Matmul->AllReduce kernels it serves live in another package.  This file is
// the Blackwell-native kernel family for them.
//
// One persistent CTA per SM, 192 threads:
//   warp 0     TMA producer: cp.async.bulk.tensor loads of A and B tiles into a
//              4-stage shared-memory ring (128-byte swizzle), completion on
//              "full" mbarriers
//   warp 1     MMA issuer: one elected thread issues tcgen05.mma
//              (cta_group::1, kind::f16, M=128, N=BN, K=16) from shared-memory
//              descriptors into one of two TMEM accumulators;
//              tcgen05.commit frees the stage ("empty") and publishes the tile
//              ("tmem full")
//   warps 2-5  epilogue: tcgen05.ld (32 lanes x 32 columns) -> registers ->
//              bf16 -> global / peer memory, overlapped with the next tile's
//              main loop through the second accumulator
// Extra CTAs beyond the GEMM CTAs act as communication workers (AllGather pull,
// ReduceScatter reduction) so that NVLink traffic overlaps the math tile by
// tile.  Remote data is never fetched by TMA with cluster multicast: peers'
// tiles are copied into this GPU's memory once (plain loads) and read from
// there by TMA, or written by plain stores.
//
// Every wait (mbarrier, local flag, peer flag) is bounded; on expiry the CTA
// raises the communicator's abort word, lets in-flight copies land, frees its
// TMEM and returns.
#pragma once
#include <cuda_bf16.h>
#include "dev_comm.cuh"
#include "reduce_ops.cuh"
#include "sm100_ptx.cuh"

namespace hccl {
namespace mc2 {

using namespace sm100;

constexpr int kBM = 128;
constexpr int kBN2c = 256;         // column tile width of the fused modes
constexpr int kBK = 64;            // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kEpilogueThreads = 128;
constexpr uint64_t kWaitLimitNs = 5ull * 1000 * 1000 * 1000;

// Epilogue staging: each of the 4 epilogue warps transposes 32 rows x 64 columns of bf16 through shared memory so
// that global / peer stores are 128 contiguous bytes per row instead of 16-byte pieces scattered over 32 rows (a
// 16-byte store is a whole NVLink packet for 16 bytes of payload).  Rows are padded by 16 bytes against bank conflicts.
constexpr int kStgRowBytes = 128 + 16;
constexpr int kStgWarpBytes = 32 * kStgRowBytes;
constexpr int kEpilogueStagingBytes = 4 * kStgWarpBytes;

enum Mode : int { MODE_PLAIN = 0, MODE_AG = 1, MODE_RS = 2, MODE_AR = 3 };

struct GemmArgs {
    // problem: C[M, N] = A[M, K] x B[K, N]   (operand storage is described by the tensor maps)
    int M, N, K;
    __nv_bfloat16* out;        // PLAIN / AG: [M, ldc]; RS: [M / P, ldc] (local reduced block); AR: [M, ldc]
    int ldc;
    int nGemmCtas;             // CTAs [0, nGemmCtas) run the GEMM; the rest are communication workers
    int tilesM, tilesN;
    // ---- fused modes
    int rank, nRanks;
    int mPerRank;              // AG: rows per rank of the gathered A; RS: rows per rank of the output
    // AG: peers' A shards (peer-mapped symmetric memory) and the local gathered buffer [P * mPerRank, K]
    const __nv_bfloat16* aPeer[kMaxDevRanks];
    __nv_bfloat16* gathered;
    // RS / AR: exchange slots.  xchg[q] = rank q's exchange buffer mapped here; layout [srcRank][rows][N] bf16
    __nv_bfloat16* xchg[kMaxDevRanks];
    // device-resident control block of the communicator's MC2 state (local memory):
    //   [0] launch epoch, [1] exit ticket, [2] abort, [16 ..) per-row-block ready counters (AG)
    uint64_t* trace;                // timeline words per CTA (kTraceWords each), filled only by builds with HCCL_MC2_TRACE
    uint32_t* ctl;
    // tile-ready flags for RS / AR: tileFlag[q] = rank q's flag array mapped here, index [srcRank][tile]
    uint64_t* tileFlag[kMaxDevRanks];
    int maxTiles;
    // The exchange buffer holds two copies of the slot array; launch L uses copy (L & 1).  A rank can only reach
    // launch L + 2 after every peer has delivered (hence started) launch L + 1, i.e. finished reading launch L, so
    // no barrier is needed before a slot is overwritten.
    size_t xchgParityElems;
    int bn;                    // two-SM kernels: column tile width (multiple of 32, at most 256), chosen per problem
    // AG, push forms (agPush != 0): `gathered` is symmetric memory, every rank stores its own shard into all ranks'
    // gathered buffers and adds the bytes written to their per-row-block arrival counters; aPeer[rank] is the local shard (any memory).
    //   gatheredPeer[q] = rank q's gathered buffer mapped here; agReady[q] = rank q's counters [P * mPerRank / 128]
    // kAgPushWorkers: dedicated worker CTAs copy; kAgPushCoop: no worker CTAs, the epilogue warps of every GEMM CTA
    // copy pieces of the shard whenever they have no accumulator to drain.
    int agPush;
    __nv_bfloat16* gatheredPeer[kMaxDevRanks];
    uint64_t* agReady[kMaxDevRanks];
    // RS, switch-reduce form (xchgMc != nullptr): every rank keeps its whole partial product [M, N] in its OWN exchange
    // buffer (local stores) and the owner of a row block reduces it with multimem.ld_reduce through the multicast
    // alias xchgMc of the exchange buffers: the partials cross NVLink inside the switch's reduction, a GPU receives
    // only its reduced block.
    const __nv_bfloat16* xchgMc;
    // plain two-SM matmul: row tiles per raster band (0 = 8) and L2 eviction policy of the operand loads
    // (0 none, 1 evict last: the operand every wave re-reads, 2 evict first: the operand that streams through once)
    int rasterGroup;
    int l2HintA, l2HintB;
    // RS without worker CTAs (rsCoop != 0): rsCoop (1 .. 4) of the epilogue warps of every GEMM CTA reduce the finished
    // tiles of this rank's row block whenever they have no accumulator to drain.  The switch-reduce path slows down
    // beyond a number of outstanding requests per GPU, so not all four warps take part by default.
    int rsCoop;
};
constexpr int kCtlEpoch = 0, kCtlTicket = 1, kCtlAbort = 2, kCtlPushNext = 3, kCtlPushGo = 4, kCtlReduceNext = 5, kCtlReady = 16;

// Timeline of a fused launch for performance work: builds with -DHCCL_MC2_TRACE (hccl_b200/build.py --trace) make
// every role of every CTA of the two-SM kernel write where its time went; other builds compile none of it.
// Absolute points are global-timer nanoseconds, durations are SM clock cycles.
enum TraceWord {
    TR_START_NS = 0, TR_GO_NS, TR_PROD_READY_CLK, TR_PROD_FIRST_REMOTE_NS, TR_PROD_EMPTY_CLK, TR_PROD_END_NS, TR_MMA_FULL_CLK, TR_MMA_TMEM_CLK,
    TR_MMA_END_NS, TR_EPI_PUSH_CLK, TR_EPI_PIECES, TR_EPI_DRAIN_CLK, TR_EPI_FULL_CLK, TR_EPI_END_NS, TR_EPI_TAIL_PUSH_CLK, TR_TILES, kTraceWords
};
#ifdef HCCL_MC2_TRACE
#define MC2_TR(...) __VA_ARGS__
#else
#define MC2_TR(...)
#endif
// agPush values
constexpr int kAgPull = 0, kAgPushWorkers = 1, kAgPushCoop = 2;

template <int BN>
struct SmemLayout {
    static constexpr int kABytes = kBM * kBK * 2;          // 16 KiB
    static constexpr int kBBytes = BN * kBK * 2;           // 32 KiB for BN = 256
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTileBytes = kStages * kStageBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kStagingOff = kTileBytes + kBarrierBytes;
    static constexpr int kTotal = kStagingOff + kEpilogueStagingBytes + 1024;   // + slack for the 1024-byte alignment
};

constexpr int kAgBandRows = 8;      // row tiles per band of the AllGather->Matmul tile order

// Flat tile index -> (m tile, n tile) in the order that suits the mode.
template <int MODE>
__device__ __forceinline__ void TileCoord(const GemmArgs& g, int t, int* mt, int* nt)
{
    if (MODE == MODE_AG) {
        // rows grouped by source rank, own rank first, then rank+1, ... : the own shard needs no transfer and the
        // gather workers fetch the others in exactly this order
        // Inside a shard: bands of up to kAgBandRows row tiles walked column by column, so that the tiles in flight
        // share a few row tiles of A AND a few column tiles of B (walking a row tile's columns first streams all of B
        // once per row tile: at a weight shard of 14336 x 8192 that alone is HBM-bound).
        const int rowTiles = g.mPerRank / kBM;
        const int tilesPerRank = rowTiles * g.tilesN;
        const int step = t / tilesPerRank, rem = t % tilesPerRank;
        const int src = (g.rank + step) % g.nRanks;
        const int band = rowTiles < kAgBandRows ? rowTiles : kAgBandRows;
        const int perBand = band * g.tilesN;
        const int first = (rem / perBand) * band, r2 = rem % perBand;
        const int rows = (rowTiles - first) < band ? (rowTiles - first) : band;
        *mt = src * rowTiles + first + r2 % rows;
        *nt = r2 / rows;
    } else if (MODE == MODE_RS) {
        // column tile major: after column tile n every rank has produced its partial of (every row block, n), so the
        // owner can reduce column tile n while the GEMM works on n + 1.  Inside a column tile the row blocks start at
        // rank + 1 so that at any time the ranks send to different owners.
        const int perCol = g.tilesM;
        const int n = t / perCol, rem = t % perCol;
        const int rowsTiles = g.mPerRank / kBM;
        const int step = rem / rowsTiles;
        const int dstRank = (g.rank + 1 + step) % g.nRanks;
        *mt = dstRank * rowsTiles + rem % rowsTiles;
        *nt = n;
    } else {
        *mt = t / g.tilesN;
        *nt = t % g.tilesN;
    }
}

__device__ __forceinline__ bool SpinUntilGE(const volatile uint32_t* p, uint32_t want, volatile uint32_t* abortWord)
{
    if (*p >= want) return true;
    const uint64_t t0 = TimerNs();
    uint32_t spins = 0;
    for (;;) {
        uint32_t v;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
        if (v >= want) return true;
        if ((++spins & 0xFFu) == 0u) {
            if (*abortWord != 0u) return false;
            if (TimerNs() - t0 > kWaitLimitNs) { *abortWord = 1u; return false; }
        }
    }
}

__device__ __forceinline__ void Store32Cols(__nv_bfloat16* dst, const uint32_t (&acc)[32], int validCols)
{
    // 32 fp32 accumulators -> 32 bf16 = 64 bytes = 4 x 16-byte stores
    uint32_t packed[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(acc[2 * i]), __uint_as_float(acc[2 * i + 1]));
        packed[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    if (validCols >= 32) {
        uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
        for (int i = 0; i < 4; ++i) d[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    } else {
        const __nv_bfloat16* e = reinterpret_cast<const __nv_bfloat16*>(packed);
        for (int i = 0; i < validCols; ++i) dst[i] = e[i];
    }
}

// Drains this warp's 32 accumulator rows x `bn` columns from TMEM and stores them as bf16 through the staging area.
// rowPtr(r, d) returns the address of column 0 of the tile in destination d for warp row r (nullptr = skip the row);
// validCols = columns of the tile that exist in the matrix.  The general form (any destination per row, several
// destinations): Matmul->AllReduce uses it; outputs with a fixed row stride take DrainTileRows below.
template <class RowPtrFn>
__device__ __forceinline__ void DrainTile(uint32_t taddrLane, int bn, uint8_t* stg, int lane, int validCols, int nDst, RowPtrFn rowPtr)
{
    for (int c0 = 0; c0 < bn; c0 += 64) {
        const int chunk = (bn - c0) < 64 ? (bn - c0) : 64;
        for (int h = 0; h < chunk; h += 32) {
            uint32_t v[32];
            TmemLd32x32(taddrLane + (uint32_t)(c0 + h), v);
            TmemLdWait();
            uint4* d = reinterpret_cast<uint4*>(stg + lane * kStgRowBytes + h * 2);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                    w[j] = *reinterpret_cast<uint32_t*>(&b);
                }
                d[i] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        __syncwarp();
        const int piecesPerRow = chunk / 8;          // 16-byte pieces
        for (int i = lane; i < 32 * piecesPerRow; i += 32) {
            const int r = i / piecesPerRow, pc = i % piecesPerRow;
            const int col = c0 + pc * 8;
            if (col >= validCols) continue;
            const uint4 val = *reinterpret_cast<const uint4*>(stg + r * kStgRowBytes + pc * 16);
            for (int dd = 0; dd < nDst; ++dd) {
                __nv_bfloat16* p = rowPtr(r, dd);
                if (p != nullptr) *reinterpret_cast<uint4*>(p + col) = val;
            }
        }
        __syncwarp();
    }
}

// Drain for destinations whose rows lie `stride` elements apart (every plain, gathered and scattered output here): the
// warp's 32 rows x `bn` columns go to base + r * stride.  Same staging as DrainTile, but the copy out of the staging
// area has no per-piece index arithmetic (DrainTile divides twice per 16-byte piece and calls a row-pointer function,
// about 150 instructions per piece: measured 12 us for a 128 x 256 tile, as long as half a main loop at an inner
// dimension of 3584): lane l always copies 16-byte column l % 8 of rows l / 8, l / 8 + 4, ..., eight loads from
// shared memory in flight, then eight stores.  The tensor-memory loads of the next 64 columns are issued before the
// copy-out and land while it runs.  validRows / validCols clip the tile at the matrix edge (columns in units of 8).
__device__ __forceinline__ void DrainTileRows(uint32_t taddrLane, int bn, uint8_t* stg, int lane, int validCols, int validRows, __nv_bfloat16* base,
                                              size_t stride)
{
    if (bn <= 0) return;
    uint32_t va[32], vb[32];
    const int pc = lane & 7, r0 = lane >> 3;
    auto issue = [&](int c0) {
        TmemLd32x32(taddrLane + (uint32_t)c0, va);
        if (bn - c0 > 32) TmemLd32x32(taddrLane + (uint32_t)(c0 + 32), vb);
    };
    auto stage = [&](const uint32_t (&v)[32], int h) {
        uint4* d = reinterpret_cast<uint4*>(stg + lane * kStgRowBytes + h * 2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                __nv_bfloat162 b = __floats2bfloat162_rn(__uint_as_float(v[8 * i + 2 * j]), __uint_as_float(v[8 * i + 2 * j + 1]));
                w[j] = *reinterpret_cast<uint32_t*>(&b);
            }
            d[i] = make_uint4(w[0], w[1], w[2], w[3]);
        }
    };
    issue(0);
    for (int c0 = 0; c0 < bn; c0 += 64) {
        const int chunk = (bn - c0) < 64 ? (bn - c0) : 64;
        TmemLdWait();
        stage(va, 0);
        if (chunk > 32) stage(vb, 32);
        __syncwarp();
        if (c0 + 64 < bn) issue(c0 + 64);
        const int col = c0 + pc * 8;
        const bool colOk = pc * 8 < chunk && col < validCols;
        uint4 v[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = *reinterpret_cast<const uint4*>(stg + (r0 + 4 * k) * kStgRowBytes + pc * 16);
        __nv_bfloat16* p = base + (size_t)r0 * stride + col;
#pragma unroll
        for (int k = 0; k < 8; ++k)
            if (colOk && r0 + 4 * k < validRows) *reinterpret_cast<uint4*>(p + (size_t)(4 * k) * stride) = v[k];
        __syncwarp();
    }
}

// -----------------------------------------------------------------------------
// Communication workers.

// AllGather pull: copies the peers' A shards into `gathered` row block by row block (kBM rows each), in the order
// rank, rank+1, rank+2, ...  One thread per worker CTA drives a ring of bulk copies (peer memory -> shared memory
// -> local memory, no multicast), kGatherStages chunks deep, so that enough bytes are in flight to cover the
// NVLink round trip; after a row block every worker adds 1 to ready[rowBlock] and a GEMM producer waits for
// ready[rowBlock] == nWorkers.  The own shard is copied the same way (the GEMM reads everything from `gathered`).
constexpr int kGatherStages = 6;
constexpr uint32_t kGatherChunk = 32 * 1024;
__device__ __forceinline__ void GatherWorker(const DevComm& c, const GemmArgs& g, int worker, int nWorkers, uint8_t* smem, uint64_t* bars)
{
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;
    const uint64_t e = LoadEpoch(c, worker);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kGatherStages; ++s) MbarInit(&bars[s], 1);
        MbarInitFence();
    }
    // peers have entered the kernel: their shards are final
    const bool ok = RankBarrier(c, worker, 0, e + 1, K_MC2_AG_GEMM);
    if (!ok && threadIdx.x == 0) *abortWord = 1u;   // the GEMM CTAs must not wait for rows that will never arrive
    if (ok && threadIdx.x == 0) {
        const size_t blockBytes = (size_t)g.K * 2 * kBM;
        const int blocksPerRank = g.mPerRank / kBM;
        const int nBlocks = g.nRanks * blocksPerRank;
        size_t b0, b1;
        Share(blockBytes, nWorkers, worker, 16, &b0, &b1);
        const size_t share = b1 - b0;
        const int chunksPerBlock = (int)((share + kGatherChunk - 1) / kGatherChunk);
        const long total = (long)chunksPerBlock * nBlocks;
        long issued = 0, stored = 0;
        bool alive = true;
        auto chunkInfo = [&](long n, const char** src, char** dst, uint32_t* bytes, int* flagIdx, bool* last) {
            const int blk = (int)(n / chunksPerBlock), ch = (int)(n % chunksPerBlock);
            // peers first, nearest consumer order; the own shard (which the GEMM reads in place) is copied last
            const int step = (blk / blocksPerRank + 1) % g.nRanks, rb = blk % blocksPerRank;
            const int srcRank = (g.rank + step) % g.nRanks;
            const size_t off = b0 + (size_t)ch * kGatherChunk;
            *bytes = (uint32_t)((share - (size_t)ch * kGatherChunk) < kGatherChunk ? (share - (size_t)ch * kGatherChunk) : kGatherChunk);
            *src = reinterpret_cast<const char*>(g.aPeer[srcRank]) + (size_t)rb * blockBytes + off;
            *dst = reinterpret_cast<char*>(g.gathered) + ((size_t)srcRank * blocksPerRank + rb) * blockBytes + off;
            *flagIdx = srcRank * blocksPerRank + rb;
            *last = ch == chunksPerBlock - 1;
        };
        while (stored < total && alive) {
            while (issued < total && issued - stored < kGatherStages) {
                const int slot = (int)(issued % kGatherStages);
                // the store that used this slot last (chunk issued - stages) must have read it out
                if (issued >= kGatherStages) BulkWaitRead((int)(stored - (issued - kGatherStages) - 1));
                const char* src; char* dst; uint32_t bytes; int fi; bool last;
                chunkInfo(issued, &src, &dst, &bytes, &fi, &last);
                MbarExpectTx(&bars[slot], bytes);
                BulkLoadG2S(smem + (size_t)slot * kGatherChunk, src, bytes, &bars[slot]);
                ++issued;
            }
            const int slot = (int)(stored % kGatherStages);
            alive = MbarWait(&bars[slot], (uint32_t)((stored / kGatherStages) & 1), abortWord, kWaitLimitNs);
            if (!alive) break;
            const char* src; char* dst; uint32_t bytes; int fi; bool last;
            chunkInfo(stored, &src, &dst, &bytes, &fi, &last);
            BulkStoreS2G(dst, smem + (size_t)slot * kGatherChunk, bytes);
            BulkCommit();
            ++stored;
            if (last) {
                BulkWaitAll();          // this worker's part of the row block is in local memory
                __threadfence();
                atomicAdd(g.ctl + kCtlReady + fi, 1u);
            }
        }
        BulkWaitAll();
        if (!alive) {
            const uint64_t t0 = TimerNs();   // loads already issued still target this CTA's shared memory
            while (TimerNs() - t0 < 200000) {}
        }
    }
    // nobody may change its shard while a peer still reads it
    RankBarrier(c, worker, 0, e + 2, K_MC2_AG_GEMM);
    StoreEpoch(c, worker, e + 2);
}

__device__ __forceinline__ bool SpinUntilGE64(const uint64_t* p, uint64_t want, volatile uint32_t* abortWord)
{
    const uint64_t t0 = TimerNs();
    uint32_t spins = 0;
    for (;;) {
        uint64_t v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
        if (v >= want) return true;
        if ((++spins & 0xFFu) == 0u) {
            if (*abortWord != 0u) return false;
            if (TimerNs() - t0 > kWaitLimitNs) { *abortWord = 1u; return false; }
        }
    }
}

// AllGather, push form.  A read over NVLink keeps few bytes in flight per SM (every request waits a round trip), a
// posted write does not, so the gather runs faster when every rank WRITES its shard to the others.  Every warp of a
// worker CTA owns one contiguous range of the local shard and copies it with plain loads and stores (16 vectors in
// flight per lane) into the gathered buffer of one destination rank after the other, nearest consumer first (rank
// r needs the shards of r, r+1, r+2, ... in this order, so this rank serves rank, rank-1, rank-2, ...).  After each
// destination the warp fences once and adds, for every 128-row block its range touches, the number of bytes it
// wrote there to the destination's arrival counter of that block; the destination's GEMM producer waits until the
// counter holds the bytes of a whole block, and the destination clears its counters when its kernel ends.  Warps
// never wait for one another, so one warp's fence (a round trip over NVLink) overlaps the other warps' copies.  One
// barrier at the start (every rank is inside the kernel: nobody still reads its gathered buffer from an earlier op
// and its counters are clear); none at the end: this rank only reads its own memory.
constexpr int kPushWarps = kThreads / 32;
__device__ __forceinline__ void GatherPushWorker(const DevComm& c, const GemmArgs& g, int worker, int nWorkers)
{
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;
    const uint64_t e = LoadEpoch(c, worker);
    const bool ok = RankBarrier(c, worker, 0, e + 1, K_MC2_AG_GEMM);
    if (!ok && threadIdx.x == 0) *abortWord = 1u;
    if (ok) {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const size_t blockBytes = (size_t)g.K * 2 * kBM;
        const int blocksPerRank = g.mPerRank / kBM;
        const size_t shardBytes = blockBytes * (size_t)blocksPerRank;
        size_t s0, s1;
        Share(shardBytes, nWorkers * kPushWarps, worker * kPushWarps + warp, 16, &s0, &s1);
        const size_t nv = (s1 - s0) >> 4;
        const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.aPeer[g.rank]) + s0);
        constexpr int U = 16;
        for (int it = 0; it < g.nRanks && nv != 0; ++it) {
            const int step = (it + 1) % g.nRanks;          // peers first; the local copy (not waited for by the GEMM) last
            const int dstRank = (g.rank - step + g.nRanks) % g.nRanks;
            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(g.gatheredPeer[dstRank]) + (size_t)g.rank * shardBytes + s0);
            for (size_t i = lane; i < nv; i += U * 32) {
                uint4 v[U];
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (i + u * 32 < nv) v[u] = __ldg(src + i + u * 32);
#pragma unroll
                for (int u = 0; u < U; ++u)
                    if (i + u * 32 < nv) dst[i + u * 32] = v[u];
            }
            __syncwarp();
            if (lane == 0) {
                __threadfence_system();
                for (size_t b = s0 / blockBytes; b * blockBytes < s1; ++b) {
                    const size_t lo = b * blockBytes > s0 ? b * blockBytes : s0;
                    const size_t hi = (b + 1) * blockBytes < s1 ? (b + 1) * blockBytes : s1;
                    uint64_t* flag = g.agReady[dstRank] + (size_t)g.rank * blocksPerRank + b;
                    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(flag), "l"((uint64_t)(hi - lo)) : "memory");
                }
            }
            __syncwarp();
        }
    }
    StoreEpoch(c, worker, e + 1);
}

// AllGather, cooperative push form.  The epilogue warps of a GEMM CTA are idle for most of a tile's main loop (a
// 256 x 256 x 8192 tile takes about 45 us, draining it a few), and a posted write needs no shared memory and almost no
// issue slots.  So instead of giving 20-28 SMs to copy workers, every CTA computes and its four epilogue warps take
// 16 KiB pieces of the local shard from a shared counter whenever no accumulator is waiting: destinations in the
// order rank-1, rank-2, ... (the order in which the consumers need this rank's rows), pieces in address order, the
// copy into this rank's own gathered buffer last.  After a piece the warp fences once and adds the bytes it wrote to
// the destination's arrival counter of every 128-row block the piece touches.  At the start of the kernel all
// epilogue warps are idle, which front-loads the transfer: the first remote rows reach their consumer long before the
// tiles of its own shard are done.  The piece size decides when the FIRST destination is complete: the ~590 epilogue
// warps of a GPU take consecutive pieces, so one round of them covers 590 x piece bytes; with 64 KiB pieces that was
// 4.6 destinations' shards at once (8 MiB each at 4096 x 8192 over 8 ranks) and the nearest consumer saw its first
// remote rows after 80-90 us, with 16 KiB pieces one round is about one shard.  One warp of CTA 0 runs the start barrier (every rank is inside the kernel: nobody
// still reads its gathered buffer from earlier work, and its arrival counters are clear) and then opens the counter.
constexpr uint32_t kPushPieceBytes = 16 * 1024;

__device__ __forceinline__ bool MbarTestWait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(SmemAddr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Run by ONE warp of CTA 0 before its tile loop.
__device__ __forceinline__ void CoopPushOpen(const DevComm& c, const GemmArgs& g, uint32_t launchEpoch, int lane)
{
    const uint64_t e = LoadEpoch(c, 0);
    bool ok = true;
    if (lane < c.nRanks) {
        StReleaseSys(FlagPtr(c, lane, 0, 0, c.rank), e + 1);
        ok = WaitFlagGE(c, FlagPtr(c, c.rank, 0, 0, lane), e + 1, K_MC2_AG_GEMM, 0, 0, lane);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
        *reinterpret_cast<volatile uint64_t*>(c.epochs) = e + 1;
        if (!ok) *(g.ctl + kCtlAbort) = 1u;          // the GEMM CTAs must not wait for rows that will never arrive
        else asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.ctl + kCtlPushGo), "r"(launchEpoch) : "memory");
    }
    __syncwarp();
}

// One piece, by one whole warp.  Returns 0 when every piece has been taken, 1 after copying one, 2 while the start
// barrier has not completed yet.
__device__ __forceinline__ int CoopPushStep(const GemmArgs& g, uint32_t launchEpoch, int lane)
{
    uint32_t go = 0, u = 0;
    if (lane == 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(go) : "l"(g.ctl + kCtlPushGo) : "memory");
    go = __shfl_sync(0xffffffffu, go, 0);
    if (go != launchEpoch) return 2;
    const size_t blockBytes = (size_t)g.K * 2 * kBM;
    const int blocksPerRank = g.mPerRank / kBM;
    const size_t shardBytes = blockBytes * (size_t)blocksPerRank;
    const uint32_t piecesPerDst = (uint32_t)((shardBytes + kPushPieceBytes - 1) / kPushPieceBytes);
    const uint32_t total = piecesPerDst * (uint32_t)g.nRanks;
    if (lane == 0) u = atomicAdd(g.ctl + kCtlPushNext, 1u);
    u = __shfl_sync(0xffffffffu, u, 0);
    if (u >= total) return 0;
    const int it = (int)(u / piecesPerDst);
    const int step = (it + 1) % g.nRanks;            // peers first, nearest consumer first; the local copy last
    const int dstRank = (g.rank - step + g.nRanks) % g.nRanks;
    const size_t s0 = (size_t)(u % piecesPerDst) * kPushPieceBytes;
    const size_t s1 = s0 + kPushPieceBytes < shardBytes ? s0 + kPushPieceBytes : shardBytes;
    const size_t nv = (s1 - s0) >> 4;                // the shard is a multiple of 16 bytes (K is a multiple of 8)
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const char*>(g.aPeer[g.rank]) + s0);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<char*>(g.gatheredPeer[dstRank]) + (size_t)g.rank * shardBytes + s0);
    // Two register buffers of 16 vectors per lane: the loads of round r + 1 are in flight while round r is stored, so
    // a warp always has 8 KiB of local reads outstanding (under the GEMM's memory traffic a load takes microseconds)
    // and never waits for a store (posted).
    constexpr int U = 16;
    const size_t rounds = (nv + U * 32 - 1) / (U * 32);
    uint4 va[U], vb[U];
    auto load = [&](uint4 (&v)[U], size_t r) {
        const size_t i = r * (U * 32) + lane;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i + k * 32 < nv) v[k] = __ldg(src + i + k * 32);
    };
    auto store = [&](const uint4 (&v)[U], size_t r) {
        const size_t i = r * (U * 32) + lane;
#pragma unroll
        for (int k = 0; k < U; ++k)
            if (i + k * 32 < nv) dst[i + k * 32] = v[k];
    };
    if (rounds > 0) load(va, 0);
    for (size_t r = 0; r < rounds; r += 2) {
        if (r + 1 < rounds) load(vb, r + 1);
        store(va, r);
        if (r + 2 < rounds) load(va, r + 2);
        if (r + 1 < rounds) store(vb, r + 1);
    }
    __syncwarp();
    if (lane == 0) {
        // One release per piece: the warp barrier above orders every lane's stores before this thread, and a release
        // at system scope is cumulative over them; a separate system fence in front of it would wait for the same
        // acknowledgements a second time (with megabytes of posted writes in flight that is about ten microseconds).
        for (size_t b = s0 / blockBytes; b * blockBytes < s1; ++b) {
            const size_t lo = b * blockBytes > s0 ? b * blockBytes : s0;
            const size_t hi = (b + 1) * blockBytes < s1 ? (b + 1) * blockBytes : s1;
            uint64_t* flag = g.agReady[dstRank] + (size_t)g.rank * blocksPerRank + b;
            asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(flag), "l"((uint64_t)(hi - lo)) : "memory");
        }
    }
    __syncwarp();
    return 1;
}

// Epilogue warp, cooperative push form: copies pieces until accumulator `bar` is ready (returns true) or no piece is
// left (returns false: the caller goes on with plain waits).
__device__ __forceinline__ bool CoopPushWhileWaiting(const GemmArgs& g, uint32_t launchEpoch, int lane, uint64_t* bar, uint32_t parity)
{
    for (;;) {
        if (MbarTestWait(bar, parity)) return true;
        const int r = CoopPushStep(g, launchEpoch, lane);
        if (r == 0) return false;
        if (r == 2 && *(volatile uint32_t*)(g.ctl + kCtlAbort) != 0u) return false;     // the plain wait that follows returns at once
    }
}

// After its last tile an epilogue warp keeps copying until the pieces run out.  Bounded: gives up when the
// communicator aborts or the start barrier stays closed for the wait limit.
__device__ __forceinline__ void CoopPushDrain(const GemmArgs& g, uint32_t launchEpoch, int lane)
{
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;
    uint64_t t0 = 0;
    for (;;) {
        const int r = CoopPushStep(g, launchEpoch, lane);
        if (r == 0) return;
        if (r == 2) {
            const uint64_t now = TimerNs();
            if (t0 == 0) t0 = now;
            if (*abortWord != 0u || now - t0 > kWaitLimitNs) return;
        }
    }
}

// One output tile of the ReduceScatter reduction: rows [mtLocal*128, +128) x cols [nt*BN, +BN), 16-byte vectors of
// 8 bf16.  U vectors of every rank's partial are requested before any is consumed (16 loads in flight per
// thread): the reduction is bound by bytes in flight from local memory, and a worker has to keep up with the tiles
// of about eight GEMM CTAs.  Partials are summed in rank order in fp32.
template <int BN, int U, int PMAX>
__device__ __forceinline__ void ReduceTile(const GemmArgs& g, const __nv_bfloat16* xbase, size_t slotElems, int mtLocal, int nt,
                                           int rowLimit, int tid, int nThreads)
{
    const int vecPerRow = BN / 8;
    const int total = kBM * vecPerRow;
    for (int v = tid; v < total; v += U * nThreads) {
        int r[U], col[U];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * nThreads;
            r[u] = mtLocal * kBM + vv / vecPerRow;
            col[u] = nt * BN + (vv % vecPerRow) * 8;
            valid[u] = vv < total && r[u] < rowLimit && col[u] < g.N;
        }
        uint4 raw[U][PMAX];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int q = 0; q < PMAX; ++q)
                if (q < g.nRanks && valid[u])
                    raw[u][q] = *reinterpret_cast<const uint4*>(xbase + (size_t)q * slotElems + (size_t)r[u] * g.N + col[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!valid[u]) continue;
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
            for (int q = 0; q < PMAX; ++q) {
                if (q < g.nRanks) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][q]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __bfloat1622float2(h[k]);
                        acc[2 * k] += f.x;
                        acc[2 * k + 1] += f.y;
                    }
                }
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
            *reinterpret_cast<uint4*>(g.out + (size_t)r[u] * g.ldc + col[u]) = o;
        }
    }
}

// One output tile reduced by the switch: rows [mtLocal*128, +128) x cols [nt*BN, +BN) of this rank's row block, read
// through the multicast alias (`mcBlock` points at this rank's row block inside it) with multimem.ld_reduce (bf16 in,
// fp32 accumulation in the switch), eight requests in flight per thread (sixteen were measured four times SLOWER:
// the switch-reduce path throttles beyond a number of outstanding requests per SM).
template <int BN>
__device__ __forceinline__ void SwitchReduceTile(const GemmArgs& g, const __nv_bfloat16* mcBlock, int mtLocal, int nt)
{
    constexpr int U = 8;
    const int vecPerRow = BN / 8;
    const int total = kBM * vecPerRow;
    for (int v = threadIdx.x; v < total; v += U * (int)blockDim.x) {
        uint4 val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * (int)blockDim.x;
            const int r = mtLocal * kBM + vv / vecPerRow, col = nt * BN + (vv % vecPerRow) * 8;
            if (vv < total && r < g.mPerRank && col < g.N) {
                const __nv_bfloat16* p = mcBlock + (size_t)r * g.N + col;
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                             : "=r"(val[u].x), "=r"(val[u].y), "=r"(val[u].z), "=r"(val[u].w)
                             : "l"(p)
                             : "memory");
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * (int)blockDim.x;
            const int r = mtLocal * kBM + vv / vecPerRow, col = nt * BN + (vv % vecPerRow) * 8;
            if (vv < total && r < g.mPerRank && col < g.N) *reinterpret_cast<uint4*>(g.out + (size_t)r * g.ldc + col) = val[u];
        }
    }
}

// ReduceScatter, cooperative form.  As with the AllGather push, the epilogue warps are idle for most of a tile's
// main loop, so they also do the reduction and every SM computes: a warp takes the next 32-row x 256-column piece of
// this rank's output (column tile major, the order in which partials complete), looks - without waiting - whether all
// ranks have published that tile, and reduces it: through the switch (multimem.ld_reduce over the ranks' exchange
// buffers) or, in the deterministic form, by summing the P partials from local memory in rank order.  A piece whose
// partials are not there yet is kept and tried again after the next look at the accumulator barrier, so a warp
// never blocks the GEMM and nothing can wait in a circle.
constexpr int kReducePieceRows = 32;

template <int PMAX>
__device__ __forceinline__ void WarpLocalReducePiece(const GemmArgs& g, const __nv_bfloat16* xbase, size_t slotElems, int row0, int col0, int lane)
{
    constexpr int U = PMAX <= 2 ? 4 : (PMAX <= 4 ? 2 : 1);          // eight local loads in flight per lane, 32 registers
    const int vecPerRow = kBN2c / 8;
    const int total = kReducePieceRows * vecPerRow;
    for (int v = lane; v < total; v += U * 32) {
        uint4 raw[U][PMAX];
        bool valid[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * 32;
            const int r = row0 + vv / vecPerRow, col = col0 + (vv % vecPerRow) * 8;
            valid[u] = vv < total && r < g.mPerRank && col < g.N;
#pragma unroll
            for (int q = 0; q < PMAX; ++q)
                if (q < g.nRanks && valid[u]) raw[u][q] = *reinterpret_cast<const uint4*>(xbase + (size_t)q * slotElems + (size_t)r * g.N + col);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!valid[u]) continue;
            const int vv = v + u * 32;
            const int r = row0 + vv / vecPerRow, col = col0 + (vv % vecPerRow) * 8;
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
            for (int q = 0; q < PMAX; ++q) {
                if (q < g.nRanks) {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][q]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __bfloat1622float2(h[k]);
                        acc[2 * k] += f.x;
                        acc[2 * k + 1] += f.y;
                    }
                }
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int k = 0; k < 4; ++k) oh[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
            *reinterpret_cast<uint4*>(g.out + (size_t)r * g.ldc + col) = o;
        }
    }
}

__device__ __forceinline__ void WarpSwitchReducePiece(const GemmArgs& g, const __nv_bfloat16* mcBlock, int row0, int col0, int lane)
{
    constexpr int U = 8;          // more outstanding switch reductions per SM were measured slower
    const int vecPerRow = kBN2c / 8;
    const int total = kReducePieceRows * vecPerRow;
    for (int v = lane; v < total; v += U * 32) {
        uint4 val[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * 32;
            const int r = row0 + vv / vecPerRow, col = col0 + (vv % vecPerRow) * 8;
            if (vv < total && r < g.mPerRank && col < g.N) {
                const __nv_bfloat16* p = mcBlock + (size_t)r * g.N + col;
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                             : "=r"(val[u].x), "=r"(val[u].y), "=r"(val[u].z), "=r"(val[u].w)
                             : "l"(p)
                             : "memory");
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int vv = v + u * 32;
            const int r = row0 + vv / vecPerRow, col = col0 + (vv % vecPerRow) * 8;
            if (vv < total && r < g.mPerRank && col < g.N) *reinterpret_cast<uint4*>(g.out + (size_t)r * g.ldc + col) = val[u];
        }
    }
}

// One step of a warp.  *pending: a piece this warp has claimed whose partials were not all there (or -1).
// Returns 0 when nothing is left for this warp, 1 after reducing a piece, 2 when its piece is not ready yet.
// Not inlined: its 16 vectors in flight must not take registers from the accumulator drain of the same warps.
static __device__ __noinline__ int CoopReduceStep(const GemmArgs& g, uint32_t launchEpoch, int lane, int* pending)
{
    const int rowsTiles = g.mPerRank / kBM;
    const int piecesPerTile = kBM / kReducePieceRows;
    const uint32_t total = (uint32_t)(rowsTiles * g.tilesN * piecesPerTile);
    int u = *pending;
    if (u < 0) {
        uint32_t t = 0;
        if (lane == 0) t = atomicAdd(g.ctl + kCtlReduceNext, 1u);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t >= total) return 0;
        u = (int)t;
    }
    const int lt = u / piecesPerTile, piece = u % piecesPerTile;
    const int nt = lt / rowsTiles, mtLocal = lt % rowsTiles;           // column tile major: the order in which partials complete
    bool ready = true;
    if (lane < g.nRanks) {
        const uint64_t* f = g.tileFlag[g.rank] + (size_t)lane * g.maxTiles + (mtLocal * g.tilesN + nt);
        uint64_t v;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(f) : "memory");
        ready = v >= (uint64_t)launchEpoch;
    }
    ready = __all_sync(0xffffffffu, ready);
    if (!ready) { *pending = u; return 2; }
    *pending = -1;
    const int row0 = mtLocal * kBM + piece * kReducePieceRows, col0 = nt * kBN2c;
    const size_t parityOff = (launchEpoch & 1u) * g.xchgParityElems;
    if (g.xchgMc != nullptr) {
        WarpSwitchReducePiece(g, g.xchgMc + parityOff + (size_t)g.rank * g.mPerRank * g.N, row0, col0, lane);
    } else {
        const __nv_bfloat16* xbase = g.xchg[g.rank] + parityOff;
        const size_t slotElems = (size_t)g.mPerRank * g.N;
        if (g.nRanks <= 2) WarpLocalReducePiece<2>(g, xbase, slotElems, row0, col0, lane);
        else if (g.nRanks <= 4) WarpLocalReducePiece<4>(g, xbase, slotElems, row0, col0, lane);
        else WarpLocalReducePiece<kMaxDevRanks>(g, xbase, slotElems, row0, col0, lane);
    }
    return 1;
}

// Reduces pieces until accumulator `bar` is ready (true) or nothing is left for this warp (false).
__device__ __forceinline__ bool CoopReduceWhileWaiting(const GemmArgs& g, uint32_t launchEpoch, int lane, int* pending, uint64_t* bar, uint32_t parity)
{
    for (;;) {
        if (MbarTestWait(bar, parity)) return true;
        const int r = CoopReduceStep(g, launchEpoch, lane, pending);
        if (r == 0) return false;
        if (r == 2 && *(volatile uint32_t*)(g.ctl + kCtlAbort) != 0u) return false;
    }
}

// After its last tile a warp reduces until the pieces run out; bounded by the wait limit per piece.
__device__ __forceinline__ void CoopReduceDrain(const GemmArgs& g, uint32_t launchEpoch, int lane, int* pending)
{
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;
    uint64_t t0 = 0;
    for (;;) {
        const int r = CoopReduceStep(g, launchEpoch, lane, pending);
        if (r == 0) return;
        if (r == 1) { t0 = 0; continue; }
        const uint64_t now = TimerNs();
        if (t0 == 0) t0 = now;
        if (*abortWord != 0u) return;
        if (now - t0 > kWaitLimitNs) { *abortWord = 1u; return; }
    }
}

// ReduceScatter reduction: for every tile of the local row block, waits until all ranks have delivered their
// partial (flag value == launch epoch), sums the P partials in rank order in fp32 and writes bf16 to `out`.
// Tiles are visited in the order they complete (column tile major).
template <int BN>
__device__ __forceinline__ void ReduceWorker(const DevComm& c, const GemmArgs& g, int worker, int nWorkers, uint64_t epoch)
{
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;
    const int rowsTiles = g.mPerRank / kBM;
    const int nLocalTiles = rowsTiles * g.tilesN;
    const size_t slotElems = (size_t)g.mPerRank * g.N;
    const __nv_bfloat16* xbase = g.xchg[g.rank] + (epoch & 1u) * g.xchgParityElems;
    for (int lt = worker; lt < nLocalTiles; lt += nWorkers) {
        const int nt = lt / rowsTiles, mtLocal = lt % rowsTiles;
        __shared__ int s_ok;
        if (threadIdx.x == 0) s_ok = 1;
        __syncthreads();
        if (threadIdx.x < g.nRanks) {
            const uint64_t* f = g.tileFlag[g.rank] + (size_t)threadIdx.x * g.maxTiles + (mtLocal * g.tilesN + nt);
            if (!WaitFlagGE(c, f, epoch, K_MC2_GEMM_RS, worker, 0, threadIdx.x)) s_ok = 0;
        }
        __syncthreads();
        if (!s_ok) break;
        if (g.xchgMc != nullptr) {
            SwitchReduceTile<BN>(g, g.xchgMc + (epoch & 1u) * g.xchgParityElems + (size_t)g.rank * g.mPerRank * g.N, mtLocal, nt);
            continue;
        }
        if (g.nRanks <= 2) ReduceTile<BN, 8, 2>(g, xbase, slotElems, mtLocal, nt, g.mPerRank, (int)threadIdx.x, (int)blockDim.x);
        else if (g.nRanks <= 4) ReduceTile<BN, 4, 4>(g, xbase, slotElems, mtLocal, nt, g.mPerRank, (int)threadIdx.x, (int)blockDim.x);
        else ReduceTile<BN, 2, kMaxDevRanks>(g, xbase, slotElems, mtLocal, nt, g.mPerRank, (int)threadIdx.x, (int)blockDim.x);
    }
    (void)abortWord;
}

// -----------------------------------------------------------------------------
template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    GemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmAOwn,
               const GemmArgs g, const DevComm c)
{
    using L = SmemLayout<BN>;
    extern __shared__ uint8_t smemRaw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smemRaw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kTileBytes);
    uint64_t* fullBar = bars;                 // [kStages]
    uint64_t* emptyBar = bars + kStages;      // [kStages]
    uint64_t* tmemFull = bars + 2 * kStages;  // [2]
    uint64_t* tmemEmpty = bars + 2 * kStages + 2;  // [2]
    uint32_t* tmemBaseSlot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    volatile uint32_t* abortWord = g.ctl + kCtlAbort;

    const int warp = threadIdx.x / 32;
    const int cta = (int)blockIdx.x;
    const uint32_t launchEpoch = *reinterpret_cast<volatile uint32_t*>(g.ctl + kCtlEpoch) + 1;   // 1, 2, 3, ...

    if (cta >= g.nGemmCtas) {
        // ---- communication worker CTA
        const int worker = cta - g.nGemmCtas, nWorkers = (int)gridDim.x - g.nGemmCtas;
        if (MODE == MODE_AG) {
            if (g.agPush) GatherPushWorker(c, g, worker, nWorkers);
            else GatherWorker(c, g, worker, nWorkers, smem, bars);
        }
        if (MODE == MODE_RS) ReduceWorker<BN>(c, g, worker, nWorkers, (uint64_t)launchEpoch);
    } else {
        // ---- GEMM CTA
        constexpr uint32_t kTmemCols = 2 * BN;       // two accumulators of BN fp32 columns
        if (threadIdx.x == 0) {
            for (int s = 0; s < kStages; ++s) { MbarInit(&fullBar[s], 1); MbarInit(&emptyBar[s], 1); }
            for (int a = 0; a < 2; ++a) { MbarInit(&tmemFull[a], 1); MbarInit(&tmemEmpty[a], kEpilogueThreads / 32); }
            MbarInitFence();
            PrefetchTensorMap(&tmA);
            PrefetchTensorMap(&tmB);
            if (MODE == MODE_AG) PrefetchTensorMap(&tmAOwn);
        }
        if (warp == 1) {
            TmemAlloc(tmemBaseSlot, kTmemCols);
            TmemRelinquish();
        }
        TcFenceBefore();
        __syncthreads();
        TcFenceAfter();
        const uint32_t tmemBase = *tmemBaseSlot;
        const int nTiles = g.tilesM * g.tilesN;
        const int kBlocks = (g.K + kBK - 1) / kBK;

        if (warp == 0) {
            // ===== TMA producer
            if (ElectOne()) {
                int stage = 0;
                uint32_t phase = 0;
                bool ok = true;
                for (int t = cta; t < nTiles && ok; t += g.nGemmCtas) {
                    int mt, nt;
                    TileCoord<MODE>(g, t, &mt, &nt);
                    // AG: rows of this rank's own shard are read from the shard itself (no wait; the copy into the
                    // gathered buffer is off the critical path), all others from the gathered buffer once they arrived
                    const int ownFirst = g.rank * (g.mPerRank / kBM);
                    const bool own = MODE == MODE_AG && mt >= ownFirst && mt < ownFirst + g.mPerRank / kBM;
                    const CUtensorMap* mapA = own ? &tmAOwn : &tmA;
                    const int rowA = (own ? mt - ownFirst : mt) * kBM;
                    if (MODE == MODE_AG && !own) {
                        const int nWorkers = (int)gridDim.x - g.nGemmCtas;
                        if (g.agPush) ok = SpinUntilGE64(g.agReady[g.rank] + mt, (uint64_t)g.K * 2 * kBM, abortWord);
                        else ok = SpinUntilGE(g.ctl + kCtlReady + mt, (uint32_t)nWorkers, abortWord);
                        FenceProxyAsync();   // reader side of the generic -> async proxy hand-over
                        if (!ok) break;
                    }
                    for (int kb = 0; kb < kBlocks; ++kb) {
                        ok = MbarWait(&emptyBar[stage], phase ^ 1u, abortWord, kWaitLimitNs);
                        if (!ok) break;
                        uint8_t* sa = smem + stage * L::kStageBytes;
                        uint8_t* sb = sa + L::kABytes;
                        MbarExpectTx(&fullBar[stage], L::kStageBytes);
                        if (!A_MN) {
                            TmaLoad2D(sa, mapA, &fullBar[stage], kb * kBK, rowA);
                        } else {
#pragma unroll
                            for (int j = 0; j < kBM / 64; ++j) TmaLoad2D(sa + j * (64 * kBK * 2), &tmA, &fullBar[stage], mt * kBM + j * 64, kb * kBK);
                        }
                        if (!B_MN) {
                            TmaLoad2D(sb, &tmB, &fullBar[stage], kb * kBK, nt * BN);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / 64; ++j) TmaLoad2D(sb + j * (64 * kBK * 2), &tmB, &fullBar[stage], nt * BN + j * 64, kb * kBK);
                        }
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                }
                if (!ok) {
                    // let copies that were already issued land before the CTA's shared memory goes away
                    const uint64_t t0 = TimerNs();
                    while (TimerNs() - t0 < 200000) {}
                }
            }
        } else if (warp == 1) {
            // ===== MMA issuer
            if (ElectOne()) {
                constexpr uint32_t idesc = InstrDescF16(kBM, BN, true, A_MN, B_MN);
                int stage = 0;
                uint32_t phase = 0;
                int acc = 0;
                uint32_t accPhase = 0;
                bool ok = true;
                for (int t = cta; t < nTiles && ok; t += g.nGemmCtas) {
                    ok = MbarWait(&tmemEmpty[acc], accPhase ^ 1u, abortWord, kWaitLimitNs);
                    if (!ok) break;
                    TcFenceAfter();
                    const uint32_t tmemD = tmemBase + (uint32_t)(acc * BN);
                    for (int kb = 0; kb < kBlocks; ++kb) {
                        ok = MbarWait(&fullBar[stage], phase, abortWord, kWaitLimitNs);
                        if (!ok) break;
                        TcFenceAfter();
                        const uint32_t sa = SmemAddr(smem + stage * L::kStageBytes);
                        const uint32_t sb = sa + L::kABytes;
                        const uint64_t da = A_MN ? SmemDescMnMajor(sa, 64 * kBK * 2) : SmemDescKMajor(sa);
                        const uint64_t db = B_MN ? SmemDescMnMajor(sb, 64 * kBK * 2) : SmemDescKMajor(sb);
#pragma unroll
                        for (int k = 0; k < kBK / kUmmaK; ++k) {
                            // K-major: 16 elements = 32 bytes along the row; MN-major: 16 K-rows of 128 bytes
                            const uint64_t aStep = (uint64_t)((A_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            const uint64_t bStep = (uint64_t)((B_MN ? kUmmaK * 128 : kUmmaK * 2) >> 4) * k;
                            UmmaF16(tmemD, da + aStep, db + bStep, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                        UmmaCommit(&emptyBar[stage]);   // the stage is free once these MMAs have read it
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                    if (!ok) break;
                    UmmaCommit(&tmemFull[acc]);
                    if (++acc == 2) { acc = 0; accPhase ^= 1u; }
                }
            }
        } else {
            // ===== epilogue warps 2..5; a warp may only touch TMEM lanes [32 * (warp % 4), +32)
            const int quarter = warp & 3;
            const int lane = threadIdx.x & 31;
            int acc = 0;
            uint32_t accPhase = 0;
            bool ok = true;
            const size_t parityOff = (launchEpoch & 1u) * g.xchgParityElems;
            bool pushLeft = MODE == MODE_AG && g.agPush == kAgPushCoop;
            bool reduceLeft = MODE == MODE_RS && (warp - 2) < g.rsCoop;      // g.rsCoop of the four epilogue warps reduce
            int reducePending = -1;
            if (pushLeft && cta == 0 && warp == 2) CoopPushOpen(c, g, launchEpoch, lane);
            for (int t = cta; t < nTiles && ok; t += g.nGemmCtas) {
                int mt, nt;
                TileCoord<MODE>(g, t, &mt, &nt);
                if (MODE == MODE_AG && pushLeft) pushLeft = CoopPushWhileWaiting(g, launchEpoch, lane, &tmemFull[acc], accPhase);
                if (MODE == MODE_RS && reduceLeft) reduceLeft = CoopReduceWhileWaiting(g, launchEpoch, lane, &reducePending, &tmemFull[acc], accPhase);
                ok = MbarWait(&tmemFull[acc], accPhase, abortWord, kWaitLimitNs);
                if (!ok) break;
                TcFenceAfter();
                const int row0 = mt * kBM + quarter * 32;
                const uint32_t taddr = tmemBase + (uint32_t)(acc * BN) + ((uint32_t)(quarter * 32) << 16);
                uint8_t* stg = smem + L::kStagingOff + quarter * kStgWarpBytes;
                const int validCols = g.N - nt * BN;
                // a warp's 32 rows lie in one rank's row block (blocks are multiples of 128 rows) and a fixed stride apart
                if (MODE == MODE_PLAIN || MODE == MODE_AG) {
                    DrainTileRows(taddr, BN, stg, lane, validCols, g.M - row0, g.out + (size_t)row0 * g.ldc + (size_t)nt * BN, (size_t)g.ldc);
                } else if (MODE == MODE_RS) {
                    // partial of row block `dst` goes into the owner's slot [me]; switch-reduce form: the partial stays in
                    // this rank's own buffer, laid out like the product
                    const int dst = row0 / g.mPerRank;
                    __nv_bfloat16* base = nullptr;
                    if (row0 < g.M && dst < g.nRanks) {
                        if (g.xchgMc != nullptr) base = g.xchg[g.rank] + parityOff + (size_t)row0 * g.N + (size_t)nt * BN;
                        else base = g.xchg[dst] + parityOff + (size_t)g.rank * g.mPerRank * g.N + (size_t)(row0 - dst * g.mPerRank) * g.N + (size_t)nt * BN;
                    }
                    DrainTileRows(taddr, BN, stg, lane, validCols, base != nullptr ? g.M - row0 : 0, base, (size_t)g.N);
                } else {
                    // AllReduce: this rank's slot on every rank
                    DrainTile(taddr, BN, stg, lane, validCols, g.nRanks, [&](int r, int dd) -> __nv_bfloat16* {
                        const int row = row0 + r;
                        if (row >= g.M) return nullptr;
                        const int dst = (g.rank + dd) % g.nRanks;
                        return g.xchg[dst] + parityOff + (size_t)g.rank * g.M * g.N + (size_t)row * g.N + (size_t)nt * BN;
                    });
                }
                // release the accumulator to the MMA warp
                TcFenceBefore();
                __syncwarp();
                if (lane == 0) MbarArrive(&tmemEmpty[acc]);
                if (++acc == 2) { acc = 0; accPhase ^= 1u; }

                if (MODE == MODE_RS || MODE == MODE_AR) {
                    // publish the tile: all 128 epilogue threads have stored, then one thread raises the flag(s)
                    // the barrier orders all epilogue threads' stores before the publishing thread, whose fence (cumulative)
                    // then covers them: one system fence per tile instead of one per thread
                    NamedBarSync(1, kEpilogueThreads);
                    const int tileId = MODE == MODE_RS ? ((mt % (g.mPerRank / kBM)) * g.tilesN + nt) : (mt * g.tilesN + nt);
                    if (MODE == MODE_RS) {
                        if (threadIdx.x == 64) {
                            const int dst = (mt * kBM) / g.mPerRank;
                            __threadfence_system();
                            StReleaseSys(g.tileFlag[dst] + (size_t)g.rank * g.maxTiles + tileId, (uint64_t)launchEpoch);
                        }
                    } else {
                        const int e = threadIdx.x - 64;
                        if (e < g.nRanks) {
                            __threadfence_system();
                            StReleaseSys(g.tileFlag[e] + (size_t)g.rank * g.maxTiles + tileId, (uint64_t)launchEpoch);
                        }
                        // AllReduce: the same CTA reduces the tile once every rank's partial is here
                        __shared__ int s_arOk;
                        if (threadIdx.x == 64) s_arOk = 1;
                        NamedBarSync(1, kEpilogueThreads);
                        if (e >= 0 && e < g.nRanks) {
                            if (!WaitFlagGE(c, g.tileFlag[g.rank] + (size_t)e * g.maxTiles + tileId, (uint64_t)launchEpoch, K_MC2_GEMM_AR, cta, 0, e))
                                s_arOk = 0;
                        }
                        NamedBarSync(1, kEpilogueThreads);
                        if (!s_arOk) { ok = false; break; }
                        {
                            // this rank's copy of every rank's partial of the tile, summed in rank order
                            const __nv_bfloat16* xb = g.xchg[g.rank] + parityOff;
                            const size_t slot = (size_t)g.M * g.N;
                            const int tid = (int)threadIdx.x - 64;
                            if (g.nRanks <= 2) ReduceTile<BN, 8, 2>(g, xb, slot, mt, nt, g.M, tid, kEpilogueThreads);
                            else if (g.nRanks <= 4) ReduceTile<BN, 4, 4>(g, xb, slot, mt, nt, g.M, tid, kEpilogueThreads);
                            else ReduceTile<BN, 2, kMaxDevRanks>(g, xb, slot, mt, nt, g.M, tid, kEpilogueThreads);
                        }
                    }
                }
            }
            if (MODE == MODE_AG && pushLeft) CoopPushDrain(g, launchEpoch, lane);
            if (MODE == MODE_RS && reduceLeft && BN == kBN2c) CoopReduceDrain(g, launchEpoch, lane, &reducePending);
        }
        // teardown: every role has left its loop (normally or by a bounded wait that ran out)
        TcFenceBefore();
        __syncthreads();
        if (warp == 1) {
            TcFenceAfter();
            TmemDealloc(tmemBase, kTmemCols);
        }
    }

    // exit ticket: the last CTA to leave advances the launch epoch and clears the AG ready counters
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
