// Memory-bound pieces of a decoder layer as single-pass sm_100a kernels (bf16 storage, fp32 math): residual add +
// RMSNorm (forward and backward), SwiGLU (forward and backward) and rotary embedding.  They replace chains of
// framework element-wise kernels around the fused matmul kernels: each tensor is read once and written once.
// The reference has no counterpart (it is a communication library); these serve the TP + SP decoder stack that the
// MC2 kernels are benchmarked in.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "hccl/hccl_fused_ops.h"
#include "../core/log.h"

namespace hccl {
namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVecPerThread = 4;          // hidden <= 256 threads * 4 vectors * 8 elements = 8192 (rows stay in registers)

__device__ __forceinline__ void Unpack8(const uint4& raw, float* f)
{
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 v = __bfloat1622float2(h[k]);
        f[2 * k] = v.x;
        f[2 * k + 1] = v.y;
    }
}
__device__ __forceinline__ uint4 Pack8(const float* f)
{
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
    return o;
}
__device__ __forceinline__ float BlockSum(float v)
{
    __shared__ float s_part[kNormThreads / 32];
    __shared__ float s_total;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    __syncthreads();                                   // s_part / s_total of an earlier call are no longer read
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = threadIdx.x < kNormThreads / 32 ? s_part[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xFFFFFFFFu, t, o);
        if (threadIdx.x == 0) s_total = t;
    }
    __syncthreads();
    return s_total;
}

// One CTA per row.  xOut = x + delta (when delta != nullptr), h = xOut * rstd * w, rstd[row] = rsqrt(mean(xOut^2) + eps).
template <int VPT>
__global__ void __launch_bounds__(kNormThreads) AddRmsNormFwdKernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                                                    const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ xOut,
                                                                    __nv_bfloat16* __restrict__ h, float* __restrict__ rstd, int hidden, float eps)
{
    const size_t row = blockIdx.x;
    const int nVec = hidden / 8;
    const uint4* xv = reinterpret_cast<const uint4*>(x + row * hidden);
    const uint4* dv = delta ? reinterpret_cast<const uint4*>(delta + row * hidden) : nullptr;
    float vals[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * kNormThreads;
        if (v < nVec) {
            Unpack8(xv[v], vals[i]);
            if (dv) {
                float d[8];
                Unpack8(dv[v], d);
#pragma unroll
                for (int k = 0; k < 8; ++k) vals[i][k] += d[k];
                // the sum is stored in bf16 and the norm is taken of the stored value, as the unfused ops would
                const uint4 packed = Pack8(vals[i]);
                reinterpret_cast<uint4*>(xOut + row * hidden)[v] = packed;
                Unpack8(packed, vals[i]);
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) ss += vals[i][k] * vals[i][k];
        }
    }
    const float r = rsqrtf(BlockSum(ss) / (float)hidden + eps);
    if (threadIdx.x == 0) rstd[row] = r;
    const uint4* wv = reinterpret_cast<const uint4*>(w);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * kNormThreads;
        if (v < nVec) {
            float wf[8], o[8];
            Unpack8(wv[v], wf);
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = vals[i][k] * r * wf[k];
            reinterpret_cast<uint4*>(h + row * hidden)[v] = Pack8(o);
        }
    }
}

// Backward of h = x * rstd * w (+ the gradient that reaches x through the residual path, dxExtra, when given):
//   dx = rstd * (dh * w) - x * rstd^3 * mean(dh * w * x) + dxExtra
//   dw = sum over rows of dh * x * rstd        (per-CTA partial sums in dwPartial[gridDim.x][hidden], fp32)
// CTA b handles rows b, b + gridDim.x, ...
template <int VPT>
__global__ void __launch_bounds__(kNormThreads) RmsNormBwdKernel(const __nv_bfloat16* __restrict__ dh, const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                                                                 const __nv_bfloat16* __restrict__ dxExtra, __nv_bfloat16* __restrict__ dx,
                                                                 float* __restrict__ dwPartial, int rows, int hidden)
{
    const int nVec = hidden / 8;
    float dwAcc[VPT][8];
#pragma unroll
    for (int i = 0; i < VPT; ++i)
#pragma unroll
        for (int k = 0; k < 8; ++k) dwAcc[i][k] = 0.f;
    for (size_t row = blockIdx.x; row < (size_t)rows; row += gridDim.x) {
        const float r = rstd[row];
        float g[VPT][8], xs[VPT][8];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * kNormThreads;
            if (v < nVec) {
                float wf[8];
                Unpack8(reinterpret_cast<const uint4*>(dh + row * hidden)[v], g[i]);
                Unpack8(reinterpret_cast<const uint4*>(x + row * hidden)[v], xs[i]);
                Unpack8(reinterpret_cast<const uint4*>(w)[v], wf);          // stays in L1 from row to row
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    dwAcc[i][k] += g[i][k] * xs[i][k] * r;
                    g[i][k] *= wf[k];
                    dot += g[i][k] * xs[i][k];
                }
            }
        }
        const float c = BlockSum(dot) / (float)hidden * r * r * r;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
            const int v = threadIdx.x + i * kNormThreads;
            if (v < nVec) {
                float o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = r * g[i][k] - xs[i][k] * c;
                if (dxExtra) {
                    float e[8];
                    Unpack8(reinterpret_cast<const uint4*>(dxExtra + row * hidden)[v], e);
#pragma unroll
                    for (int k = 0; k < 8; ++k) o[k] += e[k];
                }
                reinterpret_cast<uint4*>(dx + row * hidden)[v] = Pack8(o);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
        const int v = threadIdx.x + i * kNormThreads;
        if (v < nVec) {
            float4* p = reinterpret_cast<float4*>(dwPartial + (size_t)blockIdx.x * hidden + (size_t)v * 8);
            p[0] = make_float4(dwAcc[i][0], dwAcc[i][1], dwAcc[i][2], dwAcc[i][3]);
            p[1] = make_float4(dwAcc[i][4], dwAcc[i][5], dwAcc[i][6], dwAcc[i][7]);
        }
    }
}
__global__ void ReducePartialsKernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ dw, int nPartials, int hidden)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= hidden) return;
    float s = 0.f;
    for (int b = 0; b < nPartials; ++b) s += partial[(size_t)b * hidden + j];
    dw[j] = __float2bfloat16_rn(s);
}

// SwiGLU on gu [rows, 2 * f] (gate = columns [0, f), up = columns [f, 2f)): out = silu(gate) * up.
__global__ void SwigluFwdKernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, size_t rows, int f)
{
    const size_t nVecRow = (size_t)f / 8;
    const size_t total = rows * nVecRow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / nVecRow, v = i % nVecRow;
        float g[8], u[8], o[8];
        Unpack8(reinterpret_cast<const uint4*>(gu + row * 2 * f)[v], g);
        Unpack8(reinterpret_cast<const uint4*>(gu + row * 2 * f + f)[v], u);
#pragma unroll
        for (int k = 0; k < 8; ++k) o[k] = g[k] / (1.f + __expf(-g[k])) * u[k];
        reinterpret_cast<uint4*>(out + row * f)[v] = Pack8(o);
    }
}
__global__ void SwigluBwdKernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dgu,
                                size_t rows, int f)
{
    const size_t nVecRow = (size_t)f / 8;
    const size_t total = rows * nVecRow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / nVecRow, v = i % nVecRow;
        float g[8], u[8], d[8], dg[8], du[8];
        Unpack8(reinterpret_cast<const uint4*>(gu + row * 2 * f)[v], g);
        Unpack8(reinterpret_cast<const uint4*>(gu + row * 2 * f + f)[v], u);
        Unpack8(reinterpret_cast<const uint4*>(dout + row * f)[v], d);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float sig = 1.f / (1.f + __expf(-g[k]));
            const float silu = g[k] * sig;
            dg[k] = d[k] * u[k] * sig * (1.f + g[k] * (1.f - sig));
            du[k] = d[k] * silu;
        }
        reinterpret_cast<uint4*>(dgu + row * 2 * f)[v] = Pack8(dg);
        reinterpret_cast<uint4*>(dgu + row * 2 * f + f)[v] = Pack8(du);
    }
}

// Rotary embedding of nHeads heads of width d per row ("rotate halves": pairs (i, i + d/2)); cos / sin are fp32
// [rows, d/2].  sign = +1 forward, -1 backward (the transpose of the rotation).  Rows of `in` / `out` are inStride /
// outStride elements apart, so a slice of a wider projection output can be rotated in place or into a packed tensor.
__global__ void RopeKernel(const __nv_bfloat16* __restrict__ in, size_t inStride, __nv_bfloat16* __restrict__ out, size_t outStride,
                           const float* __restrict__ cosT, const float* __restrict__ sinT, size_t rows, int nHeads, int d, float sign)
{
    const int half = d / 2, vecHalf = half / 8;
    const size_t perRow = (size_t)nHeads * vecHalf;
    const size_t total = rows * perRow;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t row = i / perRow;
        const int rem = (int)(i % perRow), head = rem / vecHalf, v = rem % vecHalf;
        const __nv_bfloat16* src = in + row * inStride + (size_t)head * d;
        __nv_bfloat16* dst = out + row * outStride + (size_t)head * d;
        float a[8], b[8], c[8], s[8], oa[8], ob[8];
        Unpack8(reinterpret_cast<const uint4*>(src)[v], a);
        Unpack8(reinterpret_cast<const uint4*>(src + half)[v], b);
        const float4* cp = reinterpret_cast<const float4*>(cosT + row * half + (size_t)v * 8);
        const float4* sp = reinterpret_cast<const float4*>(sinT + row * half + (size_t)v * 8);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            oa[k] = a[k] * c[k] - sign * b[k] * s[k];
            ob[k] = b[k] * c[k] + sign * a[k] * s[k];
        }
        reinterpret_cast<uint4*>(dst)[v] = Pack8(oa);
        reinterpret_cast<uint4*>(dst + half)[v] = Pack8(ob);
    }
}

int VecPerThread(uint32_t hidden)
{
    const int need = (int)((hidden / 8 + kNormThreads - 1) / kNormThreads);
    return need <= 1 ? 1 : (need <= 2 ? 2 : 4);
}
bool Aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
HcclResult CheckLaunch(const char* what)
{
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { HCCL_ERROR("%s launch failed: %s", what, cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}
int ElementwiseGrid(size_t items)
{
    size_t blocks = (items + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    return blocks < 1 ? 1 : (int)blocks;
}

}  // namespace
}  // namespace hccl

using namespace hccl;

extern "C" {

HcclResult HcclFusedAddRmsNormFwd(const void* x, const void* delta, const void* w, void* xOut, void* h, void* rstd, uint64_t rows, uint32_t hidden,
                                  float eps, hcclStream_t stream)
{
    CHK_PTR_NULL(x); CHK_PTR_NULL(w); CHK_PTR_NULL(h); CHK_PTR_NULL(rstd);
    if (delta != nullptr) CHK_PTR_NULL(xOut);
    if (hidden == 0 || hidden % 8 != 0 || hidden > kNormThreads * kMaxVecPerThread * 8) return HCCL_E_PARA;
    if (!Aligned16(x) || !Aligned16(w) || !Aligned16(h) || (delta && (!Aligned16(delta) || !Aligned16(xOut)))) return HCCL_E_PARA;
    if (rows == 0) return HCCL_SUCCESS;
    const int vpt = VecPerThread(hidden);
#define HCCL_FWD(V)                                                                                                                        \
    AddRmsNormFwdKernel<V><<<(unsigned)rows, kNormThreads, 0, (cudaStream_t)stream>>>(                                                    \
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)w, (__nv_bfloat16*)xOut, (__nv_bfloat16*)h, (float*)rstd, \
        (int)hidden, eps)
    if (vpt == 1) HCCL_FWD(1); else if (vpt == 2) HCCL_FWD(2); else HCCL_FWD(4);
#undef HCCL_FWD
    return CheckLaunch("AddRmsNormFwd");
}

uint32_t HcclFusedRmsNormBwdPartials(uint64_t rows)
{
    return (uint32_t)(rows < 296 ? (rows < 1 ? 1 : rows) : 296);       // two CTAs per SM on 148 SMs
}

HcclResult HcclFusedRmsNormBwd(const void* dh, const void* x, const void* w, const void* rstd, const void* dxExtra, void* dx, void* dwPartial,
                               void* dw, uint64_t rows, uint32_t hidden, hcclStream_t stream)
{
    CHK_PTR_NULL(dh); CHK_PTR_NULL(x); CHK_PTR_NULL(w); CHK_PTR_NULL(rstd); CHK_PTR_NULL(dx); CHK_PTR_NULL(dwPartial); CHK_PTR_NULL(dw);
    if (hidden == 0 || hidden % 8 != 0 || hidden > kNormThreads * kMaxVecPerThread * 8) return HCCL_E_PARA;
    if (!Aligned16(dh) || !Aligned16(x) || !Aligned16(w) || !Aligned16(dx) || !Aligned16(dwPartial) || (dxExtra && !Aligned16(dxExtra))) return HCCL_E_PARA;
    if (rows == 0) return HCCL_SUCCESS;
    const uint32_t nPart = HcclFusedRmsNormBwdPartials(rows);
    const int vpt = VecPerThread(hidden);
#define HCCL_BWD(V)                                                                                                                         \
    RmsNormBwdKernel<V><<<nPart, kNormThreads, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dh, (const __nv_bfloat16*)x,                \
                                                                          (const __nv_bfloat16*)w, (const float*)rstd,                      \
                                                                          (const __nv_bfloat16*)dxExtra, (__nv_bfloat16*)dx,               \
                                                                          (float*)dwPartial, (int)rows, (int)hidden)
    if (vpt == 1) HCCL_BWD(1); else if (vpt == 2) HCCL_BWD(2); else HCCL_BWD(4);
#undef HCCL_BWD
    CHK_RET(CheckLaunch("RmsNormBwd"));
    ReducePartialsKernel<<<(hidden + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const float*)dwPartial, (__nv_bfloat16*)dw, (int)nPart, (int)hidden);
    return CheckLaunch("RmsNormBwd reduce");
}

HcclResult HcclFusedSwigluFwd(const void* gu, void* out, uint64_t rows, uint32_t f, hcclStream_t stream)
{
    CHK_PTR_NULL(gu); CHK_PTR_NULL(out);
    if (f == 0 || f % 8 != 0 || !Aligned16(gu) || !Aligned16(out)) return HCCL_E_PARA;
    if (rows == 0) return HCCL_SUCCESS;
    SwigluFwdKernel<<<ElementwiseGrid(rows * (f / 8)), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, rows, (int)f);
    return CheckLaunch("SwigluFwd");
}

HcclResult HcclFusedSwigluBwd(const void* gu, const void* dout, void* dgu, uint64_t rows, uint32_t f, hcclStream_t stream)
{
    CHK_PTR_NULL(gu); CHK_PTR_NULL(dout); CHK_PTR_NULL(dgu);
    if (f == 0 || f % 8 != 0 || !Aligned16(gu) || !Aligned16(dout) || !Aligned16(dgu)) return HCCL_E_PARA;
    if (rows == 0) return HCCL_SUCCESS;
    SwigluBwdKernel<<<ElementwiseGrid(rows * (f / 8)), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout,
                                                                                      (__nv_bfloat16*)dgu, rows, (int)f);
    return CheckLaunch("SwigluBwd");
}

HcclResult HcclFusedRope(const void* in, uint64_t inStride, void* out, uint64_t outStride, const void* cosTable, const void* sinTable, uint64_t rows,
                         uint32_t nHeads, uint32_t headDim, int backward, hcclStream_t stream)
{
    CHK_PTR_NULL(in); CHK_PTR_NULL(out); CHK_PTR_NULL(cosTable); CHK_PTR_NULL(sinTable);
    if (headDim == 0 || headDim % 16 != 0 || inStride % 8 != 0 || outStride % 8 != 0) return HCCL_E_PARA;
    if (!Aligned16(in) || !Aligned16(out) || !Aligned16(cosTable) || !Aligned16(sinTable)) return HCCL_E_PARA;
    if (rows == 0 || nHeads == 0) return HCCL_SUCCESS;
    RopeKernel<<<ElementwiseGrid(rows * nHeads * (headDim / 16)), 256, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)in, (size_t)inStride, (__nv_bfloat16*)out, (size_t)outStride, (const float*)cosTable, (const float*)sinTable, rows,
        (int)nHeads, (int)headDim, backward ? -1.f : 1.f);
    return CheckLaunch("Rope");
}

}  // extern "C"
