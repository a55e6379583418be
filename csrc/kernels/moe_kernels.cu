// Expert-parallel MoE dispatch and combine (sm_100a).
//
// HCCL serves MoE expert parallelism with AlltoAllV / AlltoAllVC
// (src/ops/all_to_all_v, staging protocol aiv_all_to_all_v_mesh_1D.h:105-266);
// token permutation, quantisation and the weighted sum run as separate operators
// around it.  Here the two directions are ONE kernel each:
//   dispatch  count exchange -> per (token, expert) slot assignment -> the token row is read once, quantised to
//             fp8 e4m3 with one fp32 scale per 1x128 block, and written straight into the destination rank's
//             receive buffer, grouped by local expert and, inside an expert, by source rank (ready for a grouped
//             GEMM); the variable per-peer counts never go through the host
//   combine   every rank pulls the expert outputs of its own tokens from the peers' (symmetric) output buffers and
//             accumulates sum_k gate[t, k] * y[slot(t, k)] in fp32 -> bf16, in token order: permutation back,
//             transfer and gate-weighted sum in one pass, no intermediate buffer
// Synchronisation, epochs, bounded waits: the same block-row protocol as the collectives (dev_comm.cuh).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include "coll_bodies.cuh"
#include "launch.h"
#include "moe_launch.h"
#include "../core/log.h"

namespace hccl {

namespace {

constexpr int kMoeThreads = 256;

// ------------------------------------------------------------------ count + local positions
// counts[e] = number of (token, k) pairs routed to global expert e; pos[t * K + k] = rank of the pair among this
// rank's pairs for the same expert.
__global__ void MoeCountKernel(const int32_t* __restrict__ topkIdx, int nPairs, int nExperts, uint32_t* __restrict__ counts,
                               uint32_t* __restrict__ pos)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < nPairs; i += gridDim.x * blockDim.x) {
        const int e = topkIdx[i];
        pos[i] = (e >= 0 && e < nExperts) ? atomicAdd(&counts[e], 1u) : 0xFFFFFFFFu;
    }
}

// ------------------------------------------------------------------ dispatch
struct DispatchBody {
    using Args = MoeDispatchArgs;
    static constexpr int kThreads = kMoeThreads;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        extern __shared__ uint32_t s_dyn[];   // unused: static arrays below
        __shared__ uint32_t s_cnt[kMaxDevRanks * kMoeMaxExperts];   // [src][expert]
        __shared__ uint32_t s_base[kMoeMaxExperts];                 // slot base in the destination rank for (expert, src = me)
        __shared__ float s_scale[64];                               // up to 64 blocks of 128 -> hidden <= 8192
        __shared__ uint4 s_row[8192 / 16];                          // the quantised row: hidden <= 8192 bytes of fp8
        __shared__ uint64_t s_dst[kMoeMaxTopk];                     // (destination rank, slot) of the row's copies
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const int E = a.nExperts, perRank = E / p;
        const uint64_t e0 = LoadEpoch(c, b);
        // phase 0: publish my counts in every rank's table, row `me` (each block row owns a private copy of the table)
        for (int q = 0; q < p; ++q) {
            uint32_t* tbl = a.table[q] + ((size_t)b * kMaxDevRanks + me) * kMoeMaxExperts;
            for (int e = threadIdx.x; e < E; e += blockDim.x) tbl[e] = a.counts[e];
        }
        bool ok = RankBarrier(c, b, 0, e0 + 1, K_MOE_DISPATCH);
        // phase 1: slot bases.  Destination rank d = e / perRank holds its experts one after the other; inside an expert the
        // sources are ordered by rank.
        const uint32_t* mine = a.table[me] + (size_t)b * kMaxDevRanks * kMoeMaxExperts;
        for (int i = threadIdx.x; i < p * E; i += blockDim.x) s_cnt[(i / E) * kMoeMaxExperts + (i % E)] = mine[(size_t)(i / E) * kMoeMaxExperts + (i % E)];
        __syncthreads();
        for (int e = threadIdx.x; e < E; e += blockDim.x) {
            const int d = e / perRank;
            uint32_t base = 0;
            for (int e2 = d * perRank; e2 < e; ++e2)
                for (int s = 0; s < p; ++s) base += s_cnt[s * kMoeMaxExperts + e2];
            for (int s = 0; s < me; ++s) base += s_cnt[s * kMoeMaxExperts + e];
            s_base[e] = base;
        }
        __syncthreads();
        if (b == 0) {
            // what this rank receives: per local expert total and the running offsets (for the grouped GEMM that follows)
            for (int le = threadIdx.x; le <= perRank; le += blockDim.x) {
                uint32_t off = 0;
                for (int e2 = 0; e2 < le; ++e2)
                    for (int s = 0; s < p; ++s) off += s_cnt[s * kMoeMaxExperts + me * perRank + e2];
                a.recvOffsets[le] = off;
                if (le == perRank && off > a.capacity) ReportWaitFailure(c, K_MOE_DISPATCH, b, 0, me, a.capacity, off, DEV_ERR_BOUNDS);
            }
        }
        // phase 2: token rows
        const int H = a.hidden, nScale = H / 128, vecPerRow = H / 8;      // uint4 of 8 bf16
        for (int t = b; t < a.nTokens && ok; t += nb) {
            const uint4* row = reinterpret_cast<const uint4*>(a.x + (size_t)t * H);
            // amax per 128-element block: 16 vectors per block, one vector per thread per pass
            for (int v0 = 0; v0 < vecPerRow; v0 += blockDim.x) {
                const int v = v0 + threadIdx.x;
                float amax = 0.f;
                if (v < vecPerRow) {
                    const uint4 raw = row[v];
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const float2 f = __bfloat1622float2(h[k]);
                        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
                    }
                }
                // 16 consecutive lanes cover one block of 128
#pragma unroll
                for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                if (v < vecPerRow && (threadIdx.x & 15) == 0) s_scale[v / 16] = fmaxf(amax, 1e-10f) / 448.f;
            }
            __syncthreads();
            // quantise the row ONCE into shared memory (16 bytes of fp8 = 16 elements = 2 input vectors per thread) ...
            for (int w = threadIdx.x; w < H / 16; w += blockDim.x) {
                const float inv = 1.f / s_scale[(w * 16) / 128];
                const uint4 r0 = row[2 * w], r1 = row[2 * w + 1];
                const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&r0);
                const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
                uint32_t outw[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const __nv_bfloat162* h = j < 2 ? h0 + 2 * j : h1 + 2 * (j - 2);
                    const float2 fa = __bfloat1622float2(h[0]), fb = __bfloat1622float2(h[1]);
                    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(fa.x * inv, fa.y * inv), __NV_SATFINITE, __NV_E4M3);
                    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(fb.x * inv, fb.y * inv), __NV_SATFINITE, __NV_E4M3);
                    outw[j] = (uint32_t)lo | ((uint32_t)hi << 16);
                }
                s_row[w] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
            }
            // ... and where its topk copies go
            if (threadIdx.x < a.topk) {
                const int pair = t * a.topk + threadIdx.x;
                const int e = a.topkIdx[pair];
                uint64_t sm = ~0ull;
                if (e >= 0 && e < E) sm = ((uint64_t)(e / perRank) << 32) | (uint64_t)(s_base[e] + a.pos[pair]);
                a.slotMap[pair] = sm;
                s_dst[threadIdx.x] = (sm != ~0ull && (uint32_t)sm < a.capacity) ? sm : ~0ull;      // overflow: reported by the receiver's bounds check above
            }
            __syncthreads();
            // then the K copies leave as plain stores from shared memory: every thread has all K destinations' stores of
            // its piece in flight together
            for (int w = threadIdx.x; w < H / 16; w += blockDim.x) {
                const uint4 q = s_row[w];
#pragma unroll
                for (int k = 0; k < kMoeMaxTopk; ++k) {
                    if (k >= a.topk) break;
                    const uint64_t sm = s_dst[k];
                    if (sm == ~0ull) continue;
                    reinterpret_cast<uint4*>(a.recvX[sm >> 32] + (size_t)(uint32_t)sm * H)[w] = q;
                }
            }
            for (int i = threadIdx.x; i < a.topk * nScale; i += blockDim.x) {
                const int k = i / nScale, sidx = i % nScale;
                const uint64_t sm = s_dst[k];
                if (sm != ~0ull) a.recvScale[sm >> 32][(size_t)(uint32_t)sm * nScale + sidx] = s_scale[sidx];
            }
            if (threadIdx.x < a.topk) {
                const uint64_t sm = s_dst[threadIdx.x];
                if (sm != ~0ull) a.recvSrc[sm >> 32][(uint32_t)sm] = ((uint64_t)me << 32) | (uint32_t)(t * a.topk + threadIdx.x);
            }
            __syncthreads();
        }
        RankBarrier(c, b, 0, e0 + 2, K_MOE_DISPATCH);
        StoreEpoch(c, b, e0 + 2);
        OpTail(c, b);
    }
};

// ------------------------------------------------------------------ combine
struct CombineBody {
    using Args = MoeCombineArgs;
    static constexpr int kThreads = kMoeThreads;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const uint64_t e0 = LoadEpoch(c, b);
        bool ok = RankBarrier(c, b, 0, e0 + 1, K_MOE_COMBINE);      // the peers' expert outputs are final
        const int H = a.hidden, vecPerRow = H / 8;
        // Two pieces (16 bytes each) of a token row per thread and pass: 2 x topk remote loads are requested before the
        // first is used (a pull over NVLink is bound by the bytes in flight, not by issue rate).
        constexpr int U = 2;
        for (int t = b; t < a.nTokens && ok; t += nb) {
            float w[kMoeMaxTopk];
            const __nv_bfloat16* src[kMoeMaxTopk];
#pragma unroll
            for (int k = 0; k < kMoeMaxTopk; ++k) {
                w[k] = 0.f;
                src[k] = nullptr;
                if (k < a.topk) {
                    const uint64_t sm = a.slotMap[t * a.topk + k];
                    if (sm != ~0ull && (uint32_t)sm < a.capacity) {
                        w[k] = a.topkWeight[t * a.topk + k];
                        src[k] = a.y[sm >> 32] + (size_t)(uint32_t)sm * H;
                    }
                }
            }
            for (int v0 = threadIdx.x; v0 < vecPerRow; v0 += U * blockDim.x) {
                uint4 raw[U][kMoeMaxTopk];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int v = v0 + u * blockDim.x;
#pragma unroll
                    for (int k = 0; k < kMoeMaxTopk; ++k) {
                        raw[u][k] = make_uint4(0, 0, 0, 0);
                        if (k < a.topk && v < vecPerRow && src[k] != nullptr) raw[u][k] = reinterpret_cast<const uint4*>(src[k])[v];
                    }
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const int v = v0 + u * blockDim.x;
                    if (v >= vecPerRow) continue;
                    float acc[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll
                    for (int k = 0; k < kMoeMaxTopk; ++k) {
                        if (k < a.topk) {
                            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[u][k]);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const float2 f = __bfloat1622float2(h[j]);
                                acc[2 * j] += w[k] * f.x;
                                acc[2 * j + 1] += w[k] * f.y;
                            }
                        }
                    }
                    uint4 o;
                    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                    for (int j = 0; j < 4; ++j) oh[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                    reinterpret_cast<uint4*>(a.out + (size_t)t * H)[v] = o;
                }
            }
        }
        RankBarrier(c, b, 0, e0 + 2, K_MOE_COMBINE);                 // nobody overwrites its outputs while a peer still reads
        StoreEpoch(c, b, e0 + 2);
        OpTail(c, b);
    }
};

template <class Body>
HcclResult LaunchMoe(const LaunchTarget& t, const typename Body::Args& a, int nBlocks)
{
    if (t.emu != nullptr)
        return t.emu->Post(t.emuRank, &a, sizeof(a), nBlocks, Body::kThreads, reinterpret_cast<const void*>(&CollKernelEmu<Body>), t.stream);
    CollKernel<Body><<<nBlocks, Body::kThreads, 0, t.stream>>>(*t.dev, a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("MoE kernel launch failed: %s", cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

}  // namespace

HcclResult LaunchMoeCount(const int32_t* topkIdx, int nPairs, int nExperts, uint32_t* counts, uint32_t* pos, cudaStream_t stream)
{
    CHK_CUDA(cudaMemsetAsync(counts, 0, sizeof(uint32_t) * (size_t)nExperts, stream));
    const int blocks = nPairs >= 1 << 16 ? 64 : 16;
    MoeCountKernel<<<blocks, 256, 0, stream>>>(topkIdx, nPairs, nExperts, counts, pos);
    return cudaGetLastError() == cudaSuccess ? HCCL_SUCCESS : HCCL_E_RUNTIME;
}
HcclResult LaunchMoeDispatch(const LaunchTarget& t, const MoeDispatchArgs& a, int nBlocks) { return LaunchMoe<DispatchBody>(t, a, nBlocks); }
HcclResult LaunchMoeCombine(const LaunchTarget& t, const MoeCombineArgs& a, int nBlocks) { return LaunchMoe<CombineBody>(t, a, nBlocks); }

}  // namespace hccl

// ------------------------------------------------------------------ expert offsets (local routing helper)
#include <map>
#include <mutex>
#include "moe_route.cuh"
#include "hccl/hccl_moe.h"

namespace {
constexpr uint32_t kOffsetsMaxExperts = 65536;
// scratch of HcclMoeExpertOffsets: one zero-initialised buffer per device, allocated on first use
uint32_t* OffsetsScratch()
{
    static std::mutex mu;
    static std::map<int, uint32_t*> perDev;
    std::lock_guard<std::mutex> lk(mu);
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    auto it = perDev.find(dev);
    if (it != perDev.end()) return it->second;
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, sizeof(uint32_t) * (kOffsetsMaxExperts + 1)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(uint32_t) * (kOffsetsMaxExperts + 1));
    perDev[dev] = p;
    return p;
}
}  // namespace

extern "C" HcclResult HcclMoeExpertOffsets(const int32_t* topkIdx, uint64_t nPairs, uint32_t nExperts, uint32_t* offsets, hcclStream_t stream)
{
    using namespace hccl;
    CHK_PTR_NULL(topkIdx);
    CHK_PTR_NULL(offsets);
    if (nExperts == 0 || nExperts > kOffsetsMaxExperts) { HCCL_ERROR("HcclMoeExpertOffsets: 1..%u experts supported (got %u)", kOffsetsMaxExperts, nExperts); return HCCL_E_PARA; }
    uint32_t* scratch = OffsetsScratch();
    if (!scratch) return HCCL_E_MEMORY;
    // calls that share the scratch are serialised by the stream they are issued on; use one stream per device
    MoeExpertOffsetsKernel<<<MoeExpertOffsetsBlocks(nPairs), 256, 0, (cudaStream_t)stream>>>(topkIdx, nPairs, nExperts, scratch, offsets);
    return cudaGetLastError() == cudaSuccess ? HCCL_SUCCESS : HCCL_E_RUNTIME;
}
