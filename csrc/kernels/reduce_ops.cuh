// Element types, 16-byte vector pack/unpack and the four reduction operators.
//
// Reductions accumulate 16-bit floats in fp32 (the cast is fused into the
// kernel that moves the data).  Supported reduce dtypes follow the reference
// rule set (op_common.cc:4330-4335, :4394-4396): int8/16/32/64, uint64,
// fp16/bf16/fp32/fp64; unsigned 8/16/32-bit, int128 and 8-bit floats are
// copy-only, except fp8 e4m3/e5m2 which ReduceScatter accepts (the analogue of
// the hif8 ReduceScatter kernel, aiv_reduce_scatter_mesh_1d_hif8.h).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace hccl {

enum RedOp : int { RED_SUM = 0, RED_PROD = 1, RED_MAX = 2, RED_MIN = 3 };

template <class A>
__device__ __forceinline__ A ApplyOp(A a, A b, int op)
{
    switch (op) {
        case RED_SUM: return a + b;
        case RED_PROD: return a * b;
        case RED_MAX: return a > b ? a : b;
        default: return a < b ? a : b;
    }
}

// Traits: T = storage type, Acc = accumulation type, N = elements per 16 bytes.
template <class T>
struct ElemTraits {
    using Acc = T;
    static constexpr int N = 16 / (int)sizeof(T);
    __device__ static __forceinline__ Acc Load(T v) { return v; }
    __device__ static __forceinline__ T Store(Acc v) { return v; }
};
template <>
struct ElemTraits<__half> {
    using Acc = float;
    static constexpr int N = 8;
    __device__ static __forceinline__ float Load(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half Store(float v) { return __float2half_rn(v); }
};
template <>
struct ElemTraits<__nv_bfloat16> {
    using Acc = float;
    static constexpr int N = 8;
    __device__ static __forceinline__ float Load(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 Store(float v) { return __float2bfloat16_rn(v); }
};
template <>
struct ElemTraits<__nv_fp8_e4m3> {
    using Acc = float;
    static constexpr int N = 16;
    __device__ static __forceinline__ float Load(__nv_fp8_e4m3 v) { return float(v); }
    __device__ static __forceinline__ __nv_fp8_e4m3 Store(float v) { return __nv_fp8_e4m3(v); }
};
template <>
struct ElemTraits<__nv_fp8_e5m2> {
    using Acc = float;
    static constexpr int N = 16;
    __device__ static __forceinline__ float Load(__nv_fp8_e5m2 v) { return float(v); }
    __device__ static __forceinline__ __nv_fp8_e5m2 Store(float v) { return __nv_fp8_e5m2(v); }
};

template <class T>
struct AccVec {
    typename ElemTraits<T>::Acc v[ElemTraits<T>::N];
};

template <class T>
__device__ __forceinline__ void Unpack(const uint4& raw, AccVec<T>& a)
{
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < ElemTraits<T>::N; ++i) a.v[i] = ElemTraits<T>::Load(e[i]);
}
template <class T>
__device__ __forceinline__ void Accumulate(const uint4& raw, AccVec<T>& a, int op)
{
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < ElemTraits<T>::N; ++i) a.v[i] = ApplyOp(a.v[i], ElemTraits<T>::Load(e[i]), op);
}
template <class T>
__device__ __forceinline__ uint4 Pack(const AccVec<T>& a)
{
    uint4 raw;
    T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int i = 0; i < ElemTraits<T>::N; ++i) e[i] = ElemTraits<T>::Store(a.v[i]);
    return raw;
}

__device__ __forceinline__ uint4 LdVec(const void* p)
{
    return *reinterpret_cast<const uint4*>(p);
}
__device__ __forceinline__ void StVec(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }

// Bulk byte copy by one block; handles any alignment.  All threads call it.
__device__ __forceinline__ void BlockCopyBytes(char* dst, const char* src, size_t n)
{
    if (n == 0 || dst == src) return;
    const int tid = threadIdx.x, nt = blockDim.x;
    if ((((uintptr_t)dst | (uintptr_t)src) & 15u) == 0) {
        const size_t nv = n >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(src);
        uint4* d = reinterpret_cast<uint4*>(dst);
        size_t i = tid;
        // eight loads in flight per thread: a remote copy is bound by bytes in flight, not by issue rate
        for (; i + 7 * (size_t)nt < nv; i += 8 * (size_t)nt) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = s[i + (size_t)u * nt];
#pragma unroll
            for (int u = 0; u < 8; ++u) d[i + (size_t)u * nt] = v[u];
        }
        for (; i < nv; i += nt) d[i] = s[i];
        for (size_t b = (nv << 4) + tid; b < n; b += nt) dst[b] = src[b];
    } else if ((((uintptr_t)dst ^ (uintptr_t)src) & 15u) == 0) {
        // same misalignment: scalar head up to the 16-byte boundary, vector body, scalar tail
        size_t head = (16 - ((uintptr_t)src & 15u)) & 15u;
        if (head > n) head = n;
        for (size_t b = tid; b < head; b += nt) dst[b] = src[b];
        const size_t nv = (n - head) >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(src + head);
        uint4* d = reinterpret_cast<uint4*>(dst + head);
        for (size_t i = tid; i < nv; i += nt) d[i] = s[i];
        for (size_t b = head + (nv << 4) + tid; b < n; b += nt) dst[b] = src[b];
    } else {
        // different misalignment: the loads (remote in the pull forms, a round trip each) stay 16-byte vectors from
        // the source's aligned body; only the stores (local, posted) are split to what the destination's alignment
        // allows - 4-, 2- or 1-byte pieces
        size_t head = (16 - ((uintptr_t)src & 15u)) & 15u;
        if (head > n) head = n;
        for (size_t b = tid; b < head; b += nt) dst[b] = src[b];
        const size_t nv = (n - head) >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(src + head);
        char* d = dst + head;
        const unsigned dal = (unsigned)((uintptr_t)d & 3u);
        constexpr int U = 4;
        for (size_t i = tid; i < nv; i += (size_t)U * nt) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i + (size_t)u * nt < nv) v[u] = s[i + (size_t)u * nt];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (i + (size_t)u * nt >= nv) continue;
                char* o = d + ((i + (size_t)u * nt) << 4);
                if (dal == 0) {
                    const uint32_t* w = reinterpret_cast<const uint32_t*>(&v[u]);
#pragma unroll
                    for (int k = 0; k < 4; ++k) reinterpret_cast<uint32_t*>(o)[k] = w[k];
                } else if (dal == 2) {
                    const uint16_t* w = reinterpret_cast<const uint16_t*>(&v[u]);
#pragma unroll
                    for (int k = 0; k < 8; ++k) reinterpret_cast<uint16_t*>(o)[k] = w[k];
                } else {
                    const char* w = reinterpret_cast<const char*>(&v[u]);
#pragma unroll
                    for (int k = 0; k < 16; ++k) o[k] = w[k];
                }
            }
        }
        for (size_t b = head + (nv << 4) + tid; b < n; b += nt) dst[b] = src[b];
    }
}

// Several copies at once (typically one per peer): the 512-byte pieces of all segments are dealt round-robin to the
// warps of the block, so that loads from every peer are in flight together instead of peer after peer (a sequence of
// short remote copies pays one NVLink round trip each).  Falls back to one copy after the other when a segment is not
// 16-byte aligned.
struct CopySeg {
    char* dst;
    const char* src;
    size_t bytes;
};
__device__ __forceinline__ void BlockCopyMulti(const CopySeg* segs, int n)
{
    bool aligned = true;
    size_t maxBytes = 0;
    for (int q = 0; q < n; ++q) {
        aligned = aligned && (((uintptr_t)segs[q].dst | (uintptr_t)segs[q].src) & 15u) == 0;
        maxBytes = segs[q].bytes > maxBytes ? segs[q].bytes : maxBytes;
    }
    if (!aligned || n == 1) {
        for (int q = 0; q < n; ++q) BlockCopyBytes(segs[q].dst, segs[q].src, segs[q].bytes);
        return;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nWarps = blockDim.x >> 5;
    const uint32_t chunksPerSeg = (uint32_t)((maxBytes + 511) >> 9);   // 512-byte pieces (32 lanes x 16 bytes)
    const uint32_t slots = chunksPerSeg * (uint32_t)n, un = (uint32_t)n;
    constexpr int U = 8;                                               // loads in flight per thread
    for (uint32_t slot = warp; slot < slots; slot += U * (uint32_t)nWarps) {
        uint4 v[U];
        bool ok[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t sl = slot + (uint32_t)u * nWarps;
            const uint32_t q = sl % un;
            const size_t off = ((size_t)(sl / un) << 9) + ((size_t)lane << 4);
            ok[u] = sl < slots && off + 16 <= segs[q].bytes;
            if (ok[u]) v[u] = *reinterpret_cast<const uint4*>(segs[q].src + off);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t sl = slot + (uint32_t)u * nWarps;
            const uint32_t q = sl % un;
            const size_t off = ((size_t)(sl / un) << 9) + ((size_t)lane << 4);
            if (ok[u]) *reinterpret_cast<uint4*>(segs[q].dst + off) = v[u];
        }
    }
    // tails shorter than 16 bytes
    for (int q = 0; q < n; ++q) {
        const size_t done = segs[q].bytes & ~(size_t)15;
        for (size_t b = done + threadIdx.x; b < segs[q].bytes; b += blockDim.x) segs[q].dst[b] = segs[q].src[b];
    }
}

// Remote copies plus one device-local copy in the same block.  A remote load waits a round trip over NVLink, a
// local one a fraction of that, so dealing them round-robin over the same warps would halve the remote bytes in
// flight: the last `kLocalWarps` warps take the local segment, all the others the remote ones.
constexpr int kLocalWarps = 2;
__device__ __forceinline__ void BlockCopyRemoteAndLocal(const CopySeg* remote, int nRemote, const CopySeg& local)
{
    const int nWarps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    bool aligned = ((((uintptr_t)local.dst | (uintptr_t)local.src) & 15u) == 0) && nWarps > 2 * kLocalWarps;
    for (int q = 0; q < nRemote; ++q) aligned = aligned && (((uintptr_t)remote[q].dst | (uintptr_t)remote[q].src) & 15u) == 0;
    if (!aligned || nRemote == 0 || local.bytes == 0) {
        if (nRemote > 0) BlockCopyMulti(remote, nRemote);
        BlockCopyBytes(local.dst, local.src, local.bytes);
        return;
    }
    constexpr int U = 8;
    if (warp >= nWarps - kLocalWarps) {
        const size_t nv = local.bytes >> 4;
        const uint4* s = reinterpret_cast<const uint4*>(local.src);
        uint4* d = reinterpret_cast<uint4*>(local.dst);
        const size_t st = (size_t)kLocalWarps * 32;
        size_t i = (size_t)(warp - (nWarps - kLocalWarps)) * 32 + lane;
        for (; i + (U - 1) * st < nv; i += U * st) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = s[i + u * st];
#pragma unroll
            for (int u = 0; u < U; ++u) d[i + u * st] = v[u];
        }
        for (; i < nv; i += st) d[i] = s[i];
    } else {
        const int rw = nWarps - kLocalWarps;
        size_t maxBytes = 0;
        for (int q = 0; q < nRemote; ++q) maxBytes = remote[q].bytes > maxBytes ? remote[q].bytes : maxBytes;
        const uint32_t chunksPerSeg = (uint32_t)((maxBytes + 511) >> 9);
        const uint32_t slots = chunksPerSeg * (uint32_t)nRemote, un = (uint32_t)nRemote;
        for (uint32_t slot = warp; slot < slots; slot += U * (uint32_t)rw) {
            uint4 v[U];
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t sl = slot + (uint32_t)u * rw;
                const uint32_t q = sl % un;
                const size_t off = ((size_t)(sl / un) << 9) + ((size_t)lane << 4);
                ok[u] = sl < slots && off + 16 <= remote[q].bytes;
                if (ok[u]) v[u] = *reinterpret_cast<const uint4*>(remote[q].src + off);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const uint32_t sl = slot + (uint32_t)u * rw;
                const uint32_t q = sl % un;
                const size_t off = ((size_t)(sl / un) << 9) + ((size_t)lane << 4);
                if (ok[u]) *reinterpret_cast<uint4*>(remote[q].dst + off) = v[u];
            }
        }
    }
    // tails shorter than 16 bytes
    for (size_t b = (local.bytes & ~(size_t)15) + threadIdx.x; b < local.bytes; b += blockDim.x) local.dst[b] = local.src[b];
    for (int q = 0; q < nRemote; ++q) {
        const size_t done = remote[q].bytes & ~(size_t)15;
        for (size_t b = done + threadIdx.x; b < remote[q].bytes; b += blockDim.x) remote[q].dst[b] = remote[q].src[b];
    }
}

// Contiguous share of [0, n) for part `idx` of `parts`; shares are multiples of
// `gran` except the last.
__device__ __host__ __forceinline__ void Share(size_t n, int parts, int idx, size_t gran, size_t* begin, size_t* end)
{
    size_t units = (n + gran - 1) / gran;
    size_t per = (units + parts - 1) / parts;
    size_t b = per * idx * gran, e = per * (idx + 1) * gran;
    if (b > n) b = n;
    if (e > n) e = n;
    *begin = b;
    *end = e;
}

}  // namespace hccl
