// AdamW over a list of tensors in ONE launch per 80 tensors (sm_100a, memory bound).
//
// The optimizer of the decoder-stack benchmark moves 14 bytes per bf16 parameter (read p, g, m, v; write p, m, v); a
// framework multi-tensor kernel that is launched hundreds of times with small chunks reaches about half of the HBM
// copy rate.  Here the tensor table travels in the kernel's parameter space (no device table to upload, so the launch
// can be captured in a CUDA graph as it is), a block finds its tensor by a binary search over the chunk prefix, and
// every thread keeps eight 16-byte loads in flight before the first store (32 warps per SM hide the arithmetic).
// Math is fp32 and follows torch.optim.AdamW (decoupled weight decay, bias correction, eps added after the square
// root); the square root and the division are the hardware approximations (two ulp).
// The reference has no counterpart (it is a communication library).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include "hccl/hccl_fused_ops.h"
#include "../core/log.h"

namespace hccl {
namespace {

constexpr int kAdamThreads = 256;
constexpr int kAdamMaxTensors = 80;                 // 80 * 40 B + 81 * 4 B + 4 B of the 4 KiB parameter space
constexpr uint32_t kVecPerThread = 2;                             // 8 loads in flight per thread, 64 registers: 4 blocks per SM
constexpr uint32_t kChunkVecs = kAdamThreads * kVecPerThread;     // 16-byte vectors of each array per block

struct AdamBatch {
    HcclAdamTensor t[kAdamMaxTensors];
    uint32_t chunkStart[kAdamMaxTensors + 1];       // first chunk (block) of tensor i
    uint32_t n;
};

struct AdamScalars { float lr, beta1, beta2, eps, weightDecay; };

__device__ __forceinline__ float SqrtApprox(float x)
{
    float r;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// step[0] += 1, step[1] = 1 - beta1^step, step[2] = sqrt(1 - beta2^step)
__global__ void AdamStepKernel(float* step, float beta1, float beta2)
{
    const float s = step[0] + 1.0f;
    step[0] = s;
    step[1] = 1.0f - powf(beta1, s);
    step[2] = sqrtf(1.0f - powf(beta2, s));
}

template <class T> struct Vec;
template <> struct Vec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ void Load(const uint4& raw, float* f)
    {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) { const float2 v = __bfloat1622float2(h[k]); f[2 * k] = v.x; f[2 * k + 1] = v.y; }
    }
    static __device__ __forceinline__ uint4 Store(const float* f)
    {
        uint4 o;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
        return o;
    }
    static __device__ __forceinline__ float Get(const __nv_bfloat16* p, uint64_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void Put(__nv_bfloat16* p, uint64_t i, float v) { p[i] = __float2bfloat16_rn(v); }
};
template <> struct Vec<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ void Load(const uint4& raw, float* f)
    {
        const float* h = reinterpret_cast<const float*>(&raw);
#pragma unroll
        for (int k = 0; k < 4; ++k) f[k] = h[k];
    }
    static __device__ __forceinline__ uint4 Store(const float* f)
    {
        uint4 o;
        float* h = reinterpret_cast<float*>(&o);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = f[k];
        return o;
    }
    static __device__ __forceinline__ float Get(const float* p, uint64_t i) { return p[i]; }
    static __device__ __forceinline__ void Put(float* p, uint64_t i, float v) { p[i] = v; }
};

// decay = 1 - lr * weightDecay, stepSize = lr / (1 - beta1^t), rbc2s = 1 / sqrt(1 - beta2^t): computed once per thread.
// Square root and division are the two-ulp hardware approximations; the stored values are rounded far more coarsely.
__device__ __forceinline__ void AdamElem(float& p, float g, float& m, float& v, const AdamScalars& s, float decay, float stepSize, float rbc2s)
{
    m = s.beta1 * m + (1.0f - s.beta1) * g;
    v = s.beta2 * v + (1.0f - s.beta2) * g * g;
    const float denom = SqrtApprox(v) * rbc2s + s.eps;
    p = p * decay - stepSize * __fdividef(m, denom);
}

// TP: storage type of parameters and gradients, TS: storage type of the two moments.  A block owns kChunkElems
// consecutive elements of one tensor, where an "element group" is what one 16-byte vector of the WIDER type holds.
template <class TP, class TS>
__global__ void __launch_bounds__(kAdamThreads, 4) AdamWKernel(const __grid_constant__ AdamBatch b, AdamScalars s, const float* __restrict__ step,
                                                            const float* __restrict__ lrDev)
{
    // which tensor: last i with chunkStart[i] <= blockIdx.x
    uint32_t lo = 0, hi = b.n;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (b.chunkStart[mid] <= blockIdx.x) lo = mid; else hi = mid;
    }
    const HcclAdamTensor& t = b.t[lo];
    if (lrDev) s.lr = *lrDev;
    const float decay = 1.0f - s.lr * s.weightDecay, stepSize = s.lr / step[1], rbc2s = 1.0f / step[2];
    constexpr int G = Vec<TP>::kElems < Vec<TS>::kElems ? Vec<TP>::kElems : Vec<TS>::kElems;     // elements per thread-iteration
    constexpr uint64_t kChunkElems = (uint64_t)kChunkVecs * G;
    const uint64_t begin = (uint64_t)(blockIdx.x - b.chunkStart[lo]) * kChunkElems;
    const uint64_t end = begin + kChunkElems < t.numel ? begin + kChunkElems : t.numel;
    TP* p = static_cast<TP*>(t.param);
    const TP* g = static_cast<const TP*>(t.grad);
    TS* m = static_cast<TS*>(t.expAvg);
    TS* v = static_cast<TS*>(t.expAvgSq);
    const bool aligned = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v)) & 15u) == 0;
    uint64_t done = begin;
    if (aligned && Vec<TP>::kElems == Vec<TS>::kElems) {
        // same width for all four arrays: whole 16-byte vectors, all loads of the thread before the first store
        const uint64_t nVec = (end - begin) / G;
        const uint4* pv = reinterpret_cast<const uint4*>(p + begin);
        const uint4* gv = reinterpret_cast<const uint4*>(g + begin);
        const uint4* mv = reinterpret_cast<const uint4*>(m + begin);
        const uint4* vv = reinterpret_cast<const uint4*>(v + begin);
        uint4 rp[kVecPerThread], rg[kVecPerThread], rm[kVecPerThread], rv[kVecPerThread];
#pragma unroll
        for (uint32_t k = 0; k < kVecPerThread; ++k) {
            const uint64_t i = threadIdx.x + (uint64_t)k * kAdamThreads;
            if (i < nVec) { rp[k] = pv[i]; rg[k] = __ldcs(gv + i); rm[k] = mv[i]; rv[k] = vv[i]; }
        }
#pragma unroll
        for (uint32_t k = 0; k < kVecPerThread; ++k) {
            const uint64_t i = threadIdx.x + (uint64_t)k * kAdamThreads;
            if (i >= nVec) continue;
            float fp[G], fg[G], fm[G], fv[G];
            Vec<TP>::Load(rp[k], fp);
            Vec<TP>::Load(rg[k], fg);
            Vec<TS>::Load(rm[k], fm);
            Vec<TS>::Load(rv[k], fv);
#pragma unroll
            for (int e = 0; e < G; ++e) AdamElem(fp[e], fg[e], fm[e], fv[e], s, decay, stepSize, rbc2s);
            reinterpret_cast<uint4*>(p + begin)[i] = Vec<TP>::Store(fp);
            reinterpret_cast<uint4*>(m + begin)[i] = Vec<TS>::Store(fm);
            reinterpret_cast<uint4*>(v + begin)[i] = Vec<TS>::Store(fv);
        }
        done = begin + nVec * G;
    }
    if constexpr (sizeof(TP) == 2 && sizeof(TS) == 4) {
        // bf16 parameters with fp32 moments: four elements per step, 8-byte vectors of p and g, 16-byte vectors of m and v
        if (aligned) {
            const uint64_t nGrp = (end - begin) / 4;
            const uint2* pv = reinterpret_cast<const uint2*>(p + begin);
            const uint2* gv = reinterpret_cast<const uint2*>(g + begin);
            const uint4* mv = reinterpret_cast<const uint4*>(m + begin);
            const uint4* vv = reinterpret_cast<const uint4*>(v + begin);
            uint2 rp[kVecPerThread], rg[kVecPerThread];
            uint4 rm[kVecPerThread], rv[kVecPerThread];
#pragma unroll
            for (uint32_t k = 0; k < kVecPerThread; ++k) {
                const uint64_t i = threadIdx.x + (uint64_t)k * kAdamThreads;
                if (i < nGrp) { rp[k] = pv[i]; rg[k] = __ldcs(gv + i); rm[k] = mv[i]; rv[k] = vv[i]; }
            }
#pragma unroll
            for (uint32_t k = 0; k < kVecPerThread; ++k) {
                const uint64_t i = threadIdx.x + (uint64_t)k * kAdamThreads;
                if (i >= nGrp) continue;
                float fp[4], fg[4], fm[4], fv[4];
                const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(&rp[k]);
                const __nv_bfloat162* hg = reinterpret_cast<const __nv_bfloat162*>(&rg[k]);
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const float2 a = __bfloat1622float2(hp[e]), c = __bfloat1622float2(hg[e]);
                    fp[2 * e] = a.x; fp[2 * e + 1] = a.y; fg[2 * e] = c.x; fg[2 * e + 1] = c.y;
                }
                Vec<float>::Load(rm[k], fm);
                Vec<float>::Load(rv[k], fv);
#pragma unroll
                for (int e = 0; e < 4; ++e) AdamElem(fp[e], fg[e], fm[e], fv[e], s, decay, stepSize, rbc2s);
                uint2 op;
                __nv_bfloat162* ho = reinterpret_cast<__nv_bfloat162*>(&op);
                ho[0] = __floats2bfloat162_rn(fp[0], fp[1]);
                ho[1] = __floats2bfloat162_rn(fp[2], fp[3]);
                reinterpret_cast<uint2*>(p + begin)[i] = op;
                reinterpret_cast<uint4*>(m + begin)[i] = Vec<float>::Store(fm);
                reinterpret_cast<uint4*>(v + begin)[i] = Vec<float>::Store(fv);
            }
            done = begin + nGrp * 4;
        }
    }
    // unaligned tensors and the ragged tail: element by element
    for (uint64_t i = done + threadIdx.x; i < end; i += kAdamThreads) {
        float fp = Vec<TP>::Get(p, i), fm = Vec<TS>::Get(m, i), fv = Vec<TS>::Get(v, i);
        AdamElem(fp, Vec<TP>::Get(g, i), fm, fv, s, decay, stepSize, rbc2s);
        Vec<TP>::Put(p, i, fp);
        Vec<TS>::Put(m, i, fm);
        Vec<TS>::Put(v, i, fv);
    }
}

template <class TP, class TS>
HcclResult LaunchAdam(const HcclAdamTensor* tensors, uint32_t nTensors, const AdamScalars& s, const float* step, const float* lrDev, cudaStream_t stream)
{
    constexpr int G = Vec<TP>::kElems < Vec<TS>::kElems ? Vec<TP>::kElems : Vec<TS>::kElems;
    constexpr uint64_t kChunkElems = (uint64_t)kChunkVecs * G;
    for (uint32_t first = 0; first < nTensors;) {
        AdamBatch b;
        b.n = 0;
        uint64_t chunks = 0;
        while (first < nTensors && b.n < (uint32_t)kAdamMaxTensors) {
            const HcclAdamTensor& t = tensors[first];
            if (t.numel == 0) { ++first; continue; }
            if (!t.param || !t.grad || !t.expAvg || !t.expAvgSq) return HCCL_E_PTR;
            const uint64_t c = (t.numel + kChunkElems - 1) / kChunkElems;
            if (chunks + c > 0x7FFFFFFFull) { if (b.n == 0) return HCCL_E_PARA; break; }     // next launch takes it
            b.t[b.n] = t;
            b.chunkStart[b.n] = (uint32_t)chunks;
            chunks += c;
            ++b.n;
            ++first;
        }
        if (b.n == 0) break;
        b.chunkStart[b.n] = (uint32_t)chunks;
        AdamWKernel<TP, TS><<<(unsigned)chunks, kAdamThreads, 0, stream>>>(b, s, step, lrDev);
        if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    }
    return HCCL_SUCCESS;
}

}  // namespace
}  // namespace hccl

using namespace hccl;

extern "C" HcclResult HcclFusedAdamW(const HcclAdamTensor* tensors, uint32_t nTensors, HcclDataType paramType, HcclDataType stateType, float lr,
                                     const float* lrDev, float beta1, float beta2, float eps, float weightDecay, float* stepState, hcclStream_t stream)
{
    CHK_PTR_NULL(stepState);
    if (nTensors == 0) return HCCL_SUCCESS;
    CHK_PTR_NULL(tensors);
    if (!(beta1 >= 0.f && beta1 < 1.f) || !(beta2 >= 0.f && beta2 < 1.f) || !(eps >= 0.f)) return HCCL_E_PARA;
    // everything that can be refused is checked before the step counter moves: a call that fails leaves no trace
    const bool known = (paramType == HCCL_DATA_TYPE_BFP16 && (stateType == HCCL_DATA_TYPE_BFP16 || stateType == HCCL_DATA_TYPE_FP32)) ||
                       (paramType == HCCL_DATA_TYPE_FP32 && stateType == HCCL_DATA_TYPE_FP32);
    if (!known) {
        HCCL_ERROR("HcclFusedAdamW: parameters %d with moments %d are not supported (bf16/bf16, fp32/fp32, bf16/fp32)", (int)paramType, (int)stateType);
        return HCCL_E_NOT_SUPPORT;
    }
    for (uint32_t i = 0; i < nTensors; ++i)
        if (tensors[i].numel != 0 && (!tensors[i].param || !tensors[i].grad || !tensors[i].expAvg || !tensors[i].expAvgSq)) return HCCL_E_PTR;
    cudaStream_t s = (cudaStream_t)stream;
    AdamStepKernel<<<1, 1, 0, s>>>(stepState, beta1, beta2);
    if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    const AdamScalars sc{lr, beta1, beta2, eps, weightDecay};
    if (paramType == HCCL_DATA_TYPE_BFP16 && stateType == HCCL_DATA_TYPE_BFP16) return LaunchAdam<__nv_bfloat16, __nv_bfloat16>(tensors, nTensors, sc, stepState, lrDev, s);
    if (paramType == HCCL_DATA_TYPE_FP32 && stateType == HCCL_DATA_TYPE_FP32) return LaunchAdam<float, float>(tensors, nTensors, sc, stepState, lrDev, s);
    if (paramType == HCCL_DATA_TYPE_BFP16 && stateType == HCCL_DATA_TYPE_FP32) return LaunchAdam<__nv_bfloat16, float>(tensors, nTensors, sc, stepState, lrDev, s);
    HCCL_ERROR("HcclFusedAdamW: parameters %d with moments %d are not supported (bf16/bf16, fp32/fp32, bf16/fp32)", (int)paramType, (int)stateType);
    return HCCL_E_NOT_SUPPORT;
}

extern "C" uint32_t HcclFusedAdamWLaunches(uint32_t nTensors) { return nTensors == 0 ? 0 : 1 + (nTensors + kAdamMaxTensors - 1) / kAdamMaxTensors; }
