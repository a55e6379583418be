// Instantiation, tensor-map encoding and launch of the MC2 kernels (sm_100a).
#include "mc2_launch.h"
#include <map>
#include <mutex>
#include <string>
#include <vector>
#include "../core/comm.h"
#include "../core/cuda_driver.h"
#include "../core/log.h"
#include "mc2_gemm_2sm_wide.cuh"

namespace hccl {

using namespace mc2;

Mc2State::~Mc2State()
{
    if (ctl) cudaFree(ctl);
    if (resCtxDev) cudaFree(resCtxDev);
    SymFree(&flags);
    SymFree(&xchg);
}

namespace {

static_assert(kGatherStages * (int)kGatherChunk <= SmemLayout<256>::kTileBytes, "gather ring must fit the GEMM tile ring");

// Tensor map of a row-major bf16 matrix [rows, cols] (cols contiguous) with a box of boxCols x boxRows and the
// 128-byte swizzle the UMMA descriptors assume.
HcclResult MakeMap(CUtensorMap* map, const void* ptr, uint64_t rows, uint64_t cols, uint32_t boxRows, uint32_t boxCols)
{
    const DriverApi* d = GetDriverApi();
    if (!d) return HCCL_E_DRV;
    if ((((uintptr_t)ptr) & 15u) != 0 || (cols * 2) % 16 != 0) {
        HCCL_ERROR("matmul operand %p [%llu x %llu] must be 16-byte aligned with a row pitch that is a multiple of 16 bytes", ptr,
                   (unsigned long long)rows, (unsigned long long)cols);
        return HCCL_E_PARA;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {boxCols, boxRows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = d->cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { HCCL_ERROR("cuTensorMapEncodeTiled failed: %s", DriverErrorString(r)); return HCCL_E_DRV; }
    return HCCL_SUCCESS;
}

// A: logical [M, K].  transA == 0: stored [M, K] (K-major).  transA == 1: stored [K, M] (MN-major).
HcclResult MapA(CUtensorMap* map, const void* a, uint64_t m, uint64_t k, bool mnMajor)
{
    return mnMajor ? MakeMap(map, a, k, m, kBK, 64) : MakeMap(map, a, m, k, kBM, kBK);
}
// B: logical [K, N].  transB == 1: stored [N, K] (K-major).  transB == 0: stored [K, N] (MN-major).
HcclResult MapB(CUtensorMap* map, const void* b, uint64_t n, uint64_t k, bool mnMajor, int bn)
{
    return mnMajor ? MakeMap(map, b, k, n, kBK, 64) : MakeMap(map, b, n, k, (uint32_t)bn, kBK);
}

int SmCount()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

template <int BN, bool A_MN, bool B_MN, int MODE>
HcclResult LaunchGemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const DevComm& c, int grid, bool cooperative,
                      cudaStream_t stream, const CUtensorMap* taOwn = nullptr)
{
    const CUtensorMap& ta2 = taOwn != nullptr ? *taOwn : ta;      // AG: this rank's own shard, read where it is
    auto kernel = GemmKernel<BN, A_MN, B_MN, MODE>;
    static bool attrSet = false;
    if (!attrSet) {
        CHK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout<BN>::kTotal));
        attrSet = true;
    }
    if (cooperative) {
        void* args[5] = {(void*)&ta, (void*)&tb, (void*)&ta2, (void*)&g, (void*)&c};
        cudaError_t e = cudaLaunchCooperativeKernel((const void*)kernel, dim3((unsigned)grid), dim3(kThreads), args, SmemLayout<BN>::kTotal, stream);
        if (e != cudaSuccess) { HCCL_ERROR("fused matmul launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
        return HCCL_SUCCESS;
    }
    kernel<<<grid, kThreads, SmemLayout<BN>::kTotal, stream>>>(ta, tb, ta2, g, c);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("matmul launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

template <bool A_MN, bool B_MN, int MODE>
HcclResult LaunchGemm2Sm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const DevComm& c, int grid, bool cooperative,
                         cudaStream_t stream, const CUtensorMap* taOwn = nullptr)
{
    const CUtensorMap& ta2 = taOwn != nullptr ? *taOwn : ta;
    auto kernel = GemmKernel2Sm<A_MN, B_MN, MODE>;
    static bool attrSet = false;
    if (!attrSet) {
        CHK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayout2::kTotal));
        attrSet = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = SmemLayout2::kTotal;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeCooperative;
    attrs[0].val.cooperative = cooperative ? 1 : 0;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, ta2, g, c);
    if (e != cudaSuccess) { HCCL_ERROR("two-SM matmul launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

template <bool A_MN, bool B_MN>
HcclResult LaunchGemm2SmWide(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int grid, cudaStream_t stream)
{
    auto kernel = GemmKernel2SmWide<A_MN, B_MN>;
    static bool attrSet = false;
    if (!attrSet) {
        CHK_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SmemLayoutWide::kTotal));
        attrSet = true;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = SmemLayoutWide::kTotal;
    cfg.stream = stream;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, ta, tb, g);
    if (e != cudaSuccess) { HCCL_ERROR("wide two-SM matmul launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

// Wide tiles (two column tiles per CTA pair, see mc2_gemm_2sm_wide.cuh): HCCL_MC2_WIDE=1 whenever the shape allows,
// HCCL_MC2_WIDE=auto when the inner dimension is long and there are enough tiles to fill the last wave; off otherwise.
// Measured on the decoder's matmuls the unoverlapped epilogue (about 9 us per 256 accumulator columns) costs more
// than the saved L2 traffic returns, so the double-buffered 256 x 256 kernel stays the default.
int WideMode()
{
    static int v = -2;
    if (v == -2) {
        const char* e = getenv("HCCL_MC2_WIDE");
        v = e == nullptr ? 0 : (e[0] == 'a' ? -1 : (e[0] == '1' ? 1 : 0));
    }
    return v;
}

template <int MODE>
HcclResult DispatchLayout2Sm(bool aMn, bool bMn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const DevComm& c, int grid,
                             bool coop, cudaStream_t s, const CUtensorMap* taOwn = nullptr)
{
    if (!aMn && !bMn) return LaunchGemm2Sm<false, false, MODE>(ta, tb, g, c, grid, coop, s, taOwn);
    if (!aMn && bMn) return LaunchGemm2Sm<false, true, MODE>(ta, tb, g, c, grid, coop, s, taOwn);
    if (MODE == MODE_PLAIN) {
        if (aMn && !bMn) return LaunchGemm2Sm<true, false, MODE_PLAIN>(ta, tb, g, c, grid, coop, s);
        return LaunchGemm2Sm<true, true, MODE_PLAIN>(ta, tb, g, c, grid, coop, s);
    }
    HCCL_ERROR("fused matmul kernels take A in row-major [M, K] form only");
    return HCCL_E_NOT_SUPPORT;
}

// The two-SM (cta_group::2) kernels are the default for tiles of 256 x 256; HCCL_MC2_2SM=0 keeps the one-SM kernels.
bool Use2Sm()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("HCCL_MC2_2SM");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v == 1;
}

// CTAs of a fused launch that move data instead of computing, taken from the GEMM.  HCCL_MC2_AG_WORKERS /
// HCCL_MC2_RS_WORKERS fix the counts (even, 2 .. 64); otherwise:
int ForcedWorkers(bool gather)
{
    static int forced[2] = {-1, -1};
    int& f = forced[gather ? 1 : 0];
    if (f < 0) {
        f = 0;
        const char* e = getenv(gather ? "HCCL_MC2_AG_WORKERS" : "HCCL_MC2_RS_WORKERS");
        if (e != nullptr) {
            const int n = atoi(e) & ~1;
            if (n >= 2 && n <= 64) f = n;
        }
    }
    return f;
}

// Gather workers of AllGather->Matmul are bound by bytes in flight per SM: measured at 8 ranks, 28 workers beat 20 by
// 11 % although the GEMM then needs one wave more, so they take about one SM in five.
int GatherWorkerCtas(int /*tiles*/, int /*ctasPerTile*/)
{
    if (ForcedWorkers(true) > 0) return ForcedWorkers(true);
    const int sms = SmCount() & ~1;
    return std::max(2, sms / 5) & ~1;
}

// Reduce workers of Matmul->ReduceScatter have to finish an output tile in the time the GEMM produces one for them.
// Measured under the GEMM's memory traffic: about 11.5 us per 128 x 256 tile through the switch, about 4.5 us x (P + 1)
// when the P partials are read from local memory; a wave of 256 x 256 GEMM tiles takes about 5 ns x K.  The count
// minimises max(GEMM time, reduction time) inside SMs/9 .. SMs/3; ties go to the fewer workers.
int ReduceWorkerCtas(int gemmTiles, int ctasPerTile, int localTiles128, int k, int nRanks, bool switchReduce)
{
    if (ForcedWorkers(false) > 0) return ForcedWorkers(false);
    const int sms = SmCount() & ~1;
    const int lo = std::max(2, sms / 9) & ~1, hi = std::max(2, sms / 3) & ~1;
    const double tTile = switchReduce ? 11.5 : 4.5 * (nRanks + 1);
    const double tWave = 5e-3 * k * (ctasPerTile == 2 ? 1.0 : 0.5);
    int best = lo;
    double bestCost = 1e30;
    for (int w = lo; w <= hi; w += 2) {
        const int slots = std::max(1, (sms - w) / ctasPerTile);
        const double gemm = (double)((gemmTiles + slots - 1) / slots) * tWave;
        const double reduce = (double)((localTiles128 + w - 1) / w) * tTile;
        const double cost = std::max(gemm, reduce) + tTile;
        if (cost < bestCost - 1e-9) { bestCost = cost; best = w; }
    }
    return best;
}

template <int BN, int MODE>
HcclResult DispatchLayout(bool aMn, bool bMn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const DevComm& c, int grid,
                          bool coop, cudaStream_t s, const CUtensorMap* taOwn = nullptr)
{
    if (!aMn && !bMn) return LaunchGemm<BN, false, false, MODE>(ta, tb, g, c, grid, coop, s, taOwn);
    if (!aMn && bMn) return LaunchGemm<BN, false, true, MODE>(ta, tb, g, c, grid, coop, s, taOwn);
    if (MODE == MODE_PLAIN) {
        if (aMn && !bMn) return LaunchGemm<BN, true, false, MODE_PLAIN>(ta, tb, g, c, grid, coop, s);
        return LaunchGemm<BN, true, true, MODE_PLAIN>(ta, tb, g, c, grid, coop, s);
    }
    HCCL_ERROR("fused matmul kernels take A in row-major [M, K] form only");
    return HCCL_E_NOT_SUPPORT;
}

// Control block for plain matmuls (no communicator): one per device, zeroed once.
uint32_t* PlainCtl()
{
    static std::mutex mu;
    static std::map<int, uint32_t*> perDev;
    std::lock_guard<std::mutex> lk(mu);
    int dev = 0;
    cudaGetDevice(&dev);
    auto it = perDev.find(dev);
    if (it != perDev.end()) return it->second;
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, kMc2CtlWords * sizeof(uint32_t)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, kMc2CtlWords * sizeof(uint32_t));
    perDev[dev] = p;
    return p;
}

HcclResult CheckShapes(uint64_t m, uint64_t n, uint64_t k)
{
    if (m == 0 || n == 0 || k == 0 || m > (1u << 30) || n > (1u << 30) || k > (1u << 30)) return HCCL_E_PARA;
    if (n % 8 != 0 || k % 8 != 0) { HCCL_ERROR("matmul needs N and K to be multiples of 8 (got N=%llu K=%llu)", (unsigned long long)n, (unsigned long long)k); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}

void FillPeers(CommImpl* comm, GemmArgs* g)
{
    Mc2State* st = comm->mc2.get();
    for (int q = 0; q < comm->nRanks; ++q) {
        g->xchg[q] = (__nv_bfloat16*)st->xchg.peer[q];
        g->tileFlag[q] = (uint64_t*)st->flags.peer[q];
    }
    g->ctl = st->ctl;
    g->maxTiles = kMc2MaxTiles;
    g->xchgParityElems = st->xchgParityBytes / 2;
    g->rank = comm->rank;
    g->nRanks = comm->nRanks;
}

}  // namespace

#ifdef HCCL_MC2_TRACE
// Trace builds only: one timeline buffer per process, dumped as JSON lines (one per CTA) for the launches
// HCCL_MC2_TRACE_FROM .. +2 of each kind into <HCCL_MC2_TRACE_FILE>.rank<r>.jsonl.
namespace {
uint64_t* TraceBuffer(int grid)
{
    static uint64_t* buf = nullptr;
    static int cap = 0;
    if (grid > cap) {
        if (buf) cudaFree(buf);
        if (cudaMalloc(&buf, (size_t)grid * mc2::kTraceWords * sizeof(uint64_t)) != cudaSuccess) { buf = nullptr; cap = 0; return nullptr; }
        cap = grid;
    }
    cudaMemset(buf, 0, (size_t)grid * mc2::kTraceWords * sizeof(uint64_t));
    return buf;
}
void TraceDump(const char* kind, int which, const GemmArgs& g, int grid, cudaStream_t stream)
{
    static int launches[4] = {0, 0, 0, 0};
    static const int from = [] { const char* e = getenv("HCCL_MC2_TRACE_FROM"); return e ? atoi(e) : 8; }();
    const char* prefix = getenv("HCCL_MC2_TRACE_FILE");
    const int n = launches[which]++;
    if (prefix == nullptr || g.trace == nullptr || n < from || n >= from + 3) return;
    cudaStreamSynchronize(stream);
    std::vector<uint64_t> h((size_t)grid * mc2::kTraceWords);
    cudaMemcpy(h.data(), g.trace, h.size() * sizeof(uint64_t), cudaMemcpyDeviceToHost);
    const std::string path = std::string(prefix) + ".rank" + std::to_string(g.rank) + ".jsonl";
    FILE* f = fopen(path.c_str(), "a");
    if (!f) return;
    for (int c = 0; c < grid; ++c) {
        fprintf(f, "{\"kind\": \"%s\", \"launch\": %d, \"rank\": %d, \"cta\": %d, \"M\": %d, \"N\": %d, \"K\": %d, \"bn\": %d, \"w\": [", kind, n, g.rank, c, g.M, g.N, g.K, g.bn);
        for (int i = 0; i < mc2::kTraceWords; ++i) fprintf(f, "%s%llu", i ? ", " : "", (unsigned long long)h[(size_t)c * mc2::kTraceWords + i]);
        fprintf(f, "]}\n");
    }
    fclose(f);
}
}  // namespace
#define MC2_TRACE_ARM(g, grid) (g).trace = TraceBuffer(grid)
#define MC2_TRACE_DUMP(kind, which, g, grid, stream) TraceDump(kind, which, g, grid, stream)
#else
#define MC2_TRACE_ARM(g, grid)
#define MC2_TRACE_DUMP(kind, which, g, grid, stream)
#endif

HcclResult Mc2EnsureState(CommImpl* comm, uint64_t parityBytes)
{
    if (comm->emulated() || comm->hostComm) return HCCL_E_NOT_SUPPORT;
    if (!comm->mc2) {
        std::shared_ptr<Mc2State> st(new Mc2State());
        CHK_CUDA(cudaMalloc(&st->ctl, kMc2CtlWords * sizeof(uint32_t)));
        CHK_CUDA(cudaMemset(st->ctl, 0, kMc2CtlWords * sizeof(uint32_t)));
        CHK_RET(SymAlloc(*comm->bs, comm->device, ((size_t)comm->nRanks * kMc2MaxTiles + kMc2AgBlocks) * sizeof(uint64_t), false, GetEnvConfig().forceIpc, &st->flags));
        comm->mc2 = std::move(st);
    }
    Mc2State* st = comm->mc2.get();
    if (parityBytes > st->xchgParityBytes) {
        // all ranks call with the same shapes, so they all grow together
        CHK_CUDA(cudaDeviceSynchronize());
        SymFree(&st->xchg);
        const uint64_t rounded = (parityBytes + (2u << 20) - 1) / (2u << 20) * (2u << 20);
        // with a multicast alias when the communicator runs NVLS: Matmul->ReduceScatter then reduces in the switch
        CHK_RET(SymAlloc(*comm->bs, comm->device, (size_t)rounded * 2, comm->nvls(), GetEnvConfig().forceIpc, &st->xchg));
        st->xchgParityBytes = rounded;
    }
    return HCCL_SUCCESS;
}

HcclResult Mc2Matmul(const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transA, int transB, cudaStream_t stream)
{
    CHK_PTR_NULL(a); CHK_PTR_NULL(b); CHK_PTR_NULL(out);
    CHK_RET(CheckShapes(m, n, k));
    const bool aMn = transA != 0, bMn = transB == 0;
    if (aMn && m % 8 != 0) return HCCL_E_PARA;
    const int tilesM = (int)((m + kBM - 1) / kBM);
    // narrow column tiles when the wide ones would leave most SMs idle
    const bool narrow = (uint64_t)tilesM * ((n + 255) / 256) < (uint64_t)SmCount() * 3 / 4;
    const int bn = narrow ? 128 : 256;
    CUtensorMap ta, tb;
    CHK_RET(MapA(&ta, a, m, k, aMn));
    CHK_RET(MapB(&tb, b, n, k, bMn, bn));
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    g.M = (int)m; g.N = (int)n; g.K = (int)k;
    g.out = (__nv_bfloat16*)out;
    g.ldc = (int)n;
    g.tilesM = tilesM;
    g.tilesN = (int)((n + bn - 1) / bn);
    g.ctl = PlainCtl();
    if (!g.ctl) return HCCL_E_MEMORY;
    g.nRanks = 1;
    const int grid = std::min(SmCount(), g.tilesM * g.tilesN);
    g.nGemmCtas = grid;
    DevComm dummy;
    memset(&dummy, 0, sizeof(dummy));
    if (bn == 256 && Use2Sm() && m >= 256) {
        // Column tile width: the widest tile is the most efficient one, but a last wave that is mostly empty costs a
        // whole tile time; pick the width that minimises (waves x width).  MN-major B is loaded in 64-column boxes, so
        // its half tile has to be a multiple of 64.
        const int pairs = (SmCount() & ~1) / 2;
        const int tilesM2 = (int)((m + 255) / 256);
        int bestBn = 256;
        double bestCost = 1e30;
        for (int cand : {256, 224, 192, 160, 128}) {
            if (bMn && (cand / 2) % 64 != 0) continue;
            const int tn = (int)((n + cand - 1) / cand);
            const int waves = (tilesM2 * tn + pairs - 1) / pairs;
            const double cost = (double)waves * (cand + 12);      // narrower tiles amortise the fixed per-tile work less well
            if (cost < bestCost - 1e-9) { bestCost = cost; bestBn = cand; }
        }
        // wide tiles: the same search over (waves x width) with two column tiles per work item
        {
            int wideBn = 0;
            double wideCost = 1e30;
            for (int cand : {256, 224, 192, 160, 128}) {
                if (bMn && (cand / 2) % 64 != 0) continue;
                const int tn = (int)((n + cand - 1) / cand);
                const int items = tilesM2 * ((tn + 1) / 2);
                const int waves = (items + pairs - 1) / pairs;
                const double cost = (double)waves * 2.0 * (cand + 12);
                if (cost < wideCost - 1e-9) { wideCost = cost; wideBn = cand; }
            }
            const int wideItems = tilesM2 * (((int)((n + wideBn - 1) / wideBn) + 1) / 2);
            const bool wideAuto = k >= 4096 && wideItems >= 4 * pairs && wideCost <= bestCost * 1.03;
            if (WideMode() != 0 && (WideMode() == 1 || wideAuto) && n > (uint64_t)wideBn) {
                g.bn = wideBn;
                g.tilesN = (int)((n + wideBn - 1) / wideBn);
                CHK_RET(MapB(&tb, b, n, k, bMn, wideBn / 2));
                const int grid2 = std::min(SmCount() & ~1, 2 * wideItems);
                g.nGemmCtas = grid2;
                if (!aMn && !bMn) return LaunchGemm2SmWide<false, false>(ta, tb, g, grid2, stream);
                if (!aMn && bMn) return LaunchGemm2SmWide<false, true>(ta, tb, g, grid2, stream);
                if (aMn && !bMn) return LaunchGemm2SmWide<true, false>(ta, tb, g, grid2, stream);
                return LaunchGemm2SmWide<true, true>(ta, tb, g, grid2, stream);
            }
        }
        g.bn = bestBn;
        g.tilesN = (int)((n + bestBn - 1) / bestBn);
        // B is split between the two CTAs of a pair: each loads half of the B rows of a tile
        CHK_RET(MapB(&tb, b, n, k, bMn, bestBn / 2));
        // Raster and L2 policy (experimental, HCCL_MC2_L2_HINTS=1).  About `pairs` tiles are in flight: r row tiles x c
        // column tiles, walking the columns of a band of r rows.  When one operand is small enough to live in L2 next
        // to the stream of the other, it is loaded "evict last", the streamed one "evict first", and the band covers
        // the whole small operand.  Measured on the decoder's matmuls it did not pay (evict-first lines of the
        // streamed operand leave before the other row tiles of the wave have read them), so it is off by default.
        static const bool l2Hints = [] { const char* e = getenv("HCCL_MC2_L2_HINTS"); return e != nullptr && e[0] == '1'; }();
        if (l2Hints) {
            const double bytesA = 2.0 * (double)m * (double)k, bytesB = 2.0 * (double)n * (double)k;
            const double fits = 72.0 * (1 << 20);
            if (bytesA <= fits && bytesB > 1.5 * bytesA) {
                g.l2HintA = 1; g.l2HintB = 2;
                g.rasterGroup = std::min(tilesM2, 32);            // all rows of A in one band: B is read once
            } else if (bytesB <= fits && bytesA > 1.5 * bytesB) {
                g.l2HintA = 2; g.l2HintB = 1;
                g.rasterGroup = std::max(1, std::min(8, pairs / std::max(1, g.tilesN)));   // all columns of B in flight together
            }
        }
        const int pairsWanted = tilesM2 * g.tilesN;
        const int grid2 = std::min(SmCount() & ~1, 2 * pairsWanted);
        g.nGemmCtas = grid2;
        return DispatchLayout2Sm<MODE_PLAIN>(aMn, bMn, ta, tb, g, dummy, grid2, false, stream);
    }
    if (bn == 128) return DispatchLayout<128, MODE_PLAIN>(aMn, bMn, ta, tb, g, dummy, grid, false, stream);
    return DispatchLayout<256, MODE_PLAIN>(aMn, bMn, ta, tb, g, dummy, grid, false, stream);
}

HcclResult Mc2AllGatherMatmul(CommImpl* comm, const void* aShard, const void* b, void* out, void* gathered, uint64_t mPerRank, uint64_t n,
                              uint64_t k, int transB, cudaStream_t stream)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(aShard); CHK_PTR_NULL(b); CHK_PTR_NULL(out); CHK_PTR_NULL(gathered);
    const uint64_t P = (uint64_t)comm->nRanks;
    CHK_RET(CheckShapes(mPerRank * P, n, k));
    if (mPerRank % kBM != 0) { HCCL_ERROR("AllGather->Matmul needs rows per rank to be a multiple of %d (got %llu)", kBM, (unsigned long long)mPerRank); return HCCL_E_PARA; }
    if (P * (mPerRank / kBM) > 8 * 512) return HCCL_E_PARA;
    // Push form when the gathered buffer is symmetric memory (every rank writes its shard into the others' buffers;
    // the shard itself may live anywhere); pull form when only the shard is.  HCCL_MC2_AG_PULL=1 keeps the pull form.
    const char* peers[kMaxDevRanks] = {nullptr};
    const char* gathPeers[kMaxDevRanks] = {nullptr};
    static const bool forcePull = [] { const char* e = getenv("HCCL_MC2_AG_PULL"); return e != nullptr && e[0] == '1'; }();
    const bool push = !forcePull && comm->Lookup(gathered, P * mPerRank * k * 2, gathPeers, nullptr);
    if (!push && !comm->Lookup(aShard, mPerRank * k * 2, peers, nullptr)) {
        HCCL_ERROR("AllGather->Matmul: the gathered buffer or the activation shard must live in symmetric memory (HcclMemAlloc)");
        return HCCL_E_PARA;
    }
    CHK_RET(Mc2EnsureState(comm, 0));
    const bool bMn = transB == 0;
    CUtensorMap ta, tb, taOwn;
    CHK_RET(MapA(&ta, gathered, mPerRank * P, k, false));
    CHK_RET(MapA(&taOwn, aShard, mPerRank, k, false));
    CHK_RET(MapB(&tb, b, n, k, bMn, 256));
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    FillPeers(comm, &g);
    g.M = (int)(mPerRank * P); g.N = (int)n; g.K = (int)k;
    g.out = (__nv_bfloat16*)out;
    g.ldc = (int)n;
    g.tilesM = g.M / kBM;
    g.tilesN = (int)((n + 255) / 256);
    g.mPerRank = (int)mPerRank;
    for (int q = 0; q < comm->nRanks; ++q) g.aPeer[q] = (const __nv_bfloat16*)peers[q];
    g.gathered = (__nv_bfloat16*)gathered;
    if (push) {
        g.agPush = kAgPushWorkers;
        g.aPeer[comm->rank] = (const __nv_bfloat16*)aShard;
        for (int q = 0; q < comm->nRanks; ++q) {
            g.gatheredPeer[q] = (__nv_bfloat16*)gathPeers[q];
            g.agReady[q] = (uint64_t*)comm->mc2->flags.peer[q] + (size_t)comm->nRanks * kMc2MaxTiles;
        }
    }
    const bool twoSm = Use2Sm() && mPerRank % 256 == 0;
    const int grid = SmCount() & ~1;
    // Push form without worker CTAs (the default): every CTA computes, its epilogue warps copy the shard while they
    // wait for accumulators.  HCCL_MC2_AG_WORKERS=<n> keeps n dedicated copy CTAs instead.
    const bool coop = push && ForcedWorkers(true) == 0;
    int workers = 0;
    if (coop) g.agPush = kAgPushCoop;
    else workers = twoSm ? GatherWorkerCtas((g.M / 256) * g.tilesN, 2) : GatherWorkerCtas(g.tilesM * g.tilesN, 1);
    g.nGemmCtas = grid - workers;
    if (twoSm) {
        // column tile width: fewest (waves x width), as for the plain matmul; MN-major B is loaded in 64-column boxes
        const int pairs = g.nGemmCtas / 2;
        const int tilesM2 = g.M / 256;
        int bestBn = 256;
        double bestCost = 1e30;
        for (int cand : {256, 224, 192, 160, 128}) {
            if (bMn && (cand / 2) % 64 != 0) continue;
            const int tn = (int)((n + cand - 1) / cand);
            const int waves = (tilesM2 * tn + pairs - 1) / pairs;
            const double cost = (double)waves * (cand + 12);
            if (cost < bestCost - 1e-9) { bestCost = cost; bestBn = cand; }
        }
        g.bn = bestBn;
        g.tilesN = (int)((n + bestBn - 1) / bestBn);
        CHK_RET(MapB(&tb, b, n, k, bMn, bestBn / 2));
        MC2_TRACE_ARM(g, grid);
        const HcclResult r = DispatchLayout2Sm<MODE_AG>(false, bMn, ta, tb, g, comm->dev(), grid, true, stream, &taOwn);
        MC2_TRACE_DUMP("ag_matmul", 0, g, grid, stream);
        return r;
    }
    return DispatchLayout<256, MODE_AG>(false, bMn, ta, tb, g, comm->dev(), grid, true, stream, &taOwn);
}

HcclResult Mc2MatmulReduceScatter(CommImpl* comm, const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transB,
                                  cudaStream_t stream)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(a); CHK_PTR_NULL(b); CHK_PTR_NULL(out);
    const uint64_t P = (uint64_t)comm->nRanks;
    CHK_RET(CheckShapes(m, n, k));
    if (m % (P * kBM) != 0) { HCCL_ERROR("Matmul->ReduceScatter needs M to be a multiple of %llu (got %llu)", (unsigned long long)(P * kBM), (unsigned long long)m); return HCCL_E_PARA; }
    const uint64_t mPerRank = m / P;
    const uint64_t tilesN = (n + 255) / 256;
    if ((mPerRank / kBM) * tilesN > (uint64_t)kMc2MaxTiles) return HCCL_E_PARA;
    CHK_RET(Mc2EnsureState(comm, P * mPerRank * n * 2));
    const bool bMn = transB == 0;
    CUtensorMap ta, tb;
    CHK_RET(MapA(&ta, a, m, k, false));
    CHK_RET(MapB(&tb, b, n, k, bMn, 256));
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    FillPeers(comm, &g);
    g.M = (int)m; g.N = (int)n; g.K = (int)k;
    g.out = (__nv_bfloat16*)out;
    g.ldc = (int)n;
    g.tilesM = (int)(m / kBM);
    g.tilesN = (int)tilesN;
    g.mPerRank = (int)mPerRank;
    // switch-reduce form unless determinism is asked for (the switch's summation order is unspecified) or
    // HCCL_MC2_RS_P2P=1 keeps the peer-to-peer form
    static const bool forceP2p = [] { const char* e = getenv("HCCL_MC2_RS_P2P"); return e != nullptr && e[0] == '1'; }();
    // ... or at two ranks, where every rank reduces half of the product and the switch form measured 0.79 ms against
    // 0.51 ms for the peer-to-peer form (HCCL_MC2_RS_P2P=0 asks for the switch form anyway)
    static const bool forceSwitch = [] { const char* e = getenv("HCCL_MC2_RS_P2P"); return e != nullptr && e[0] == '0'; }();
    if (comm->mc2->xchg.mc != nullptr && !forceP2p && comm->cfg.deterministic == Deterministic::OFF && (comm->nRanks > 2 || forceSwitch))
        g.xchgMc = (const __nv_bfloat16*)comm->mc2->xchg.mc;
    const bool twoSm = Use2Sm() && mPerRank % 256 == 0;
    const int localTiles = (int)(mPerRank / kBM) * g.tilesN;
    // No worker CTAs by default: every CTA computes, its epilogue warps reduce the finished tiles of this rank's row
    // block while they wait for accumulators.  HCCL_MC2_RS_WORKERS=<n> keeps n dedicated reduction CTAs instead.
    int workers = 0;
    static const int rsWarps = [] { const char* e = getenv("HCCL_MC2_RS_WARPS"); const int v = e ? atoi(e) : 4; return v < 1 ? 1 : (v > 4 ? 4 : v); }();
    // Every rank count: with the division-free accumulator drain the epilogue warps have the time, and at inner
    // dimensions of ten thousand and more (two-way tensor parallelism) worker CTAs only take SMs from the GEMM
    // (measured at two ranks, 4096 x 8192 x 14336: 0.64 ms against 0.71 ms with workers).
    if (ForcedWorkers(false) == 0) g.rsCoop = rsWarps;
    else workers = twoSm ? ReduceWorkerCtas((g.M / 256) * g.tilesN, 2, localTiles, g.K, g.nRanks, g.xchgMc != nullptr)
                         : ReduceWorkerCtas(g.tilesM * g.tilesN, 1, localTiles, g.K, g.nRanks, g.xchgMc != nullptr);
    const int grid = SmCount() & ~1;
    g.nGemmCtas = grid - workers;
    if (twoSm) {
        g.bn = 256;
        CHK_RET(MapB(&tb, b, n, k, bMn, 128));
        MC2_TRACE_ARM(g, grid);
        const HcclResult r = DispatchLayout2Sm<MODE_RS>(false, bMn, ta, tb, g, comm->dev(), grid, true, stream);
        MC2_TRACE_DUMP("matmul_rs", 1, g, grid, stream);
        return r;
    }
    return DispatchLayout<256, MODE_RS>(false, bMn, ta, tb, g, comm->dev(), grid, true, stream);
}

HcclResult Mc2MatmulAllReduce(CommImpl* comm, const void* a, const void* b, void* out, uint64_t m, uint64_t n, uint64_t k, int transB,
                              cudaStream_t stream)
{
    CHK_PTR_NULL(comm); CHK_PTR_NULL(a); CHK_PTR_NULL(b); CHK_PTR_NULL(out);
    const uint64_t P = (uint64_t)comm->nRanks;
    CHK_RET(CheckShapes(m, n, k));
    if (transB == 0) { HCCL_ERROR("Matmul->AllReduce takes the weight as [N, K]"); return HCCL_E_NOT_SUPPORT; }
    const int tilesM = (int)((m + kBM - 1) / kBM), tilesN = (int)((n + 127) / 128);
    if ((uint64_t)tilesM * tilesN > (uint64_t)kMc2MaxTiles) return HCCL_E_PARA;
    // every tile is reduced by the CTA that computed it, which waits for its peers: all tiles must be resident at once
    if (tilesM * tilesN > SmCount()) { HCCL_ERROR("Matmul->AllReduce handles at most %d output tiles of 128x128 (decode shapes)", SmCount()); return HCCL_E_NOT_SUPPORT; }
    CHK_RET(Mc2EnsureState(comm, P * m * n * 2));
    CUtensorMap ta, tb;
    CHK_RET(MapA(&ta, a, m, k, false));
    CHK_RET(MapB(&tb, b, n, k, false, 128));
    GemmArgs g;
    memset(&g, 0, sizeof(g));
    FillPeers(comm, &g);
    g.M = (int)m; g.N = (int)n; g.K = (int)k;
    g.out = (__nv_bfloat16*)out;
    g.ldc = (int)n;
    g.tilesM = tilesM;
    g.tilesN = tilesN;
    const int grid = tilesM * tilesN;
    g.nGemmCtas = grid;
    return LaunchGemm<128, false, false, MODE_AR>(ta, tb, g, comm->dev(), grid, true, stream);
}

}  // namespace hccl
