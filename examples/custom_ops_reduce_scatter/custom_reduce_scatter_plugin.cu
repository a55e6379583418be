// A third-party ReduceScatter (sum of fp32 / bf16) written against the public programming model only: symmetric
// windows give every peer's mapping of the send buffer, HcclBarrier orders the ranks, and an own kernel reads block
// `me` of every peer and adds the values in rank order (so the result does not depend on timing).  Packaged as an
// algorithm plugin: an unmodified HcclReduceScatter call runs it when the send buffer lies in symmetric memory
// (the counterpart of HCCL's examples/06_custom_ops_reduce_scatter).
//
// Build (from the repository root, after `python hccl_b200/build.py`):
//   nvcc -shared -Xcompiler -fPIC -std=c++17 -gencode arch=compute_100a,code=sm_100a -Icsrc/include \
//        examples/custom_ops_reduce_scatter/custom_reduce_scatter_plugin.cu -Lhccl_b200/lib -lhccl_b200 \
//        -o libcustom_reduce_scatter.so
// Use: HCCL_ALGO_PLUGIN_PATH=$PWD/libcustom_reduce_scatter.so <any program that calls HcclReduceScatter>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include "hccl/hccl.h"
#include "hccl/hccl_algo_plugin.h"
#include "hccl/hccl_comm.h"

namespace {

constexpr int kMaxRanks = 8;
struct PeerTable {
    const char* src[kMaxRanks];     // every rank's send buffer as mapped here
};

__device__ inline float4 Add(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// out[i] = sum over ranks q (in rank order) of src[q][me * count + i].  One 16-byte vector per thread and peer; the
// loads of all peers are issued before the first add so that every link has a request in flight.
template <class T>
__global__ void ReduceBlockKernel(PeerTable t, T* out, size_t count, int nRanks, int me)
{
    constexpr int kPerVec = 16 / sizeof(T);
    const size_t nv = count / kPerVec;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        uint4 v[kMaxRanks];
#pragma unroll
        for (int q = 0; q < kMaxRanks; ++q)
            if (q < nRanks) v[q] = reinterpret_cast<const uint4*>(t.src[q] + (size_t)me * count * sizeof(T))[i];
        if constexpr (sizeof(T) == 4) {
            float4 acc = *reinterpret_cast<float4*>(&v[0]);
#pragma unroll
            for (int q = 1; q < kMaxRanks; ++q)
                if (q < nRanks) acc = Add(acc, *reinterpret_cast<float4*>(&v[q]));
            reinterpret_cast<float4*>(out)[i] = acc;
        } else {
            float acc[8];
            const __nv_bfloat16* h0 = reinterpret_cast<const __nv_bfloat16*>(&v[0]);
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = __bfloat162float(h0[e]);
#pragma unroll
            for (int q = 1; q < kMaxRanks; ++q) {
                if (q >= nRanks) continue;
                const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(&v[q]);
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] += __bfloat162float(h[e]);
            }
            uint4 r;
            __nv_bfloat16* hr = reinterpret_cast<__nv_bfloat16*>(&r);
#pragma unroll
            for (int e = 0; e < 8; ++e) hr[e] = __float2bfloat16(acc[e]);
            reinterpret_cast<uint4*>(out)[i] = r;
        }
    }
    // ragged tail, element by element
    for (size_t i = nv * kPerVec + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride) {
        float acc = 0.f;
        for (int q = 0; q < nRanks; ++q) acc += (float)reinterpret_cast<const T*>(t.src[q])[(size_t)me * count + i];
        out[i] = (T)acc;
    }
}

bool Ready() { return true; }

HcclResult Select(const HcclAlgoPluginParam* p, char name[HCCL_ALGO_PLUGIN_ALG_NAME_LEN])
{
    if (p == nullptr || p->magic != HCCL_ALGO_PLUGIN_PARAM_MAGIC || strcmp(p->opName, "ReduceScatter") != 0) return HCCL_E_NOT_SUPPORT;
    if (p->reduceOp != HCCL_REDUCE_SUM || (p->dataType != HCCL_DATA_TYPE_FP32 && p->dataType != HCCL_DATA_TYPE_BFP16)) return HCCL_E_NOT_SUPPORT;
    const size_t es = p->dataType == HCCL_DATA_TYPE_FP32 ? 4 : 2;
    // the block of every rank has to start on a 16-byte boundary for the vector loads
    if (p->rankNum < 2 || p->rankNum > kMaxRanks || ((uintptr_t)p->sendBuf & 15u) || ((uintptr_t)p->recvBuf & 15u) || (p->count * es) % 16) return HCCL_E_NOT_SUPPORT;
    void* peer = nullptr;
    if (HcclCommSymWinGet(p->comm, p->sendBuf, (p->rank + 1) % p->rankNum, &peer) != HCCL_SUCCESS) return HCCL_E_NOT_SUPPORT;
    snprintf(name, HCCL_ALGO_PLUGIN_ALG_NAME_LEN, "CustomReduceScatterPull");
    return HCCL_SUCCESS;
}

HcclResult Execute(const char*, const HcclAlgoPluginParam* p)
{
    PeerTable t;
    memset(&t, 0, sizeof(t));
    for (uint32_t q = 0; q < p->rankNum; ++q) {
        void* peer = nullptr;
        HcclResult r = HcclCommSymWinGet(p->comm, p->sendBuf, q, &peer);
        if (r != HCCL_SUCCESS) return r;
        t.src[q] = (const char*)peer;
    }
    cudaStream_t stream = (cudaStream_t)p->stream;
    HcclResult r = HcclBarrier(p->comm, p->stream);           // every rank's send buffer is final
    if (r != HCCL_SUCCESS) return r;
    const size_t es = p->dataType == HCCL_DATA_TYPE_FP32 ? 4 : 2;
    size_t blocks = (p->count * es / 16 + 255) / 256;
    blocks = blocks < 1 ? 1 : (blocks > 128 ? 128 : blocks);
    if (p->dataType == HCCL_DATA_TYPE_FP32) ReduceBlockKernel<float><<<(int)blocks, 256, 0, stream>>>(t, (float*)p->recvBuf, p->count, (int)p->rankNum, (int)p->rank);
    else ReduceBlockKernel<__nv_bfloat16><<<(int)blocks, 256, 0, stream>>>(t, (__nv_bfloat16*)p->recvBuf, p->count, (int)p->rankNum, (int)p->rank);
    if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    return HcclBarrier(p->comm, p->stream);                   // nobody overwrites its send buffer before all have read it
}

HcclAlgoPluginTable g_table = {HCCL_PLUGIN_API_VERSION, HCCL_ALGO_PLUGIN_TABLE_MAGIC, sizeof(HcclAlgoPluginTable), Ready, Select, Execute};

}  // namespace

extern "C" const HcclAlgoPluginTable* GetHcclAlgoPlugin(void) { return &g_table; }
