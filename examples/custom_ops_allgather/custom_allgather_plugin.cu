// A third-party AllGather written against the public programming model only: symmetric windows
// (HcclMemAlloc / HcclCommSymWinGet give the peers' mappings of a buffer), HcclBarrier for cross-rank ordering and
// an own CUDA kernel that pulls the peers' blocks.  It is packaged as an algorithm plugin, so an unmodified
// HcclAllGather call runs it (the counterpart of HCCL's examples/05_custom_ops_allgather, which shows the same
// thing for its three engines).
//
// Build (from the repository root, after `python hccl_b200/build.py`):
//   nvcc -shared -Xcompiler -fPIC -std=c++17 -gencode arch=compute_100a,code=sm_100a -Icsrc/include \
//        examples/custom_ops_allgather/custom_allgather_plugin.cu -Lhccl_b200/lib -lhccl_b200 -o libcustom_allgather.so
// Use: HCCL_ALGO_PLUGIN_PATH=$PWD/libcustom_allgather.so <any program that calls HcclAllGather>
// The plugin claims AllGather calls whose send buffer lies in symmetric memory; every other call (and every other
// operator) falls through to the built-in algorithms.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstring>
#include "hccl/hccl.h"
#include "hccl/hccl_algo_plugin.h"
#include "hccl/hccl_comm.h"

namespace {

constexpr int kMaxRanks = 8;
struct PeerTable {
    const char* src[kMaxRanks];
};

// Block q of the output = rank q's send buffer.  Sixteen-byte vectors, eight loads in flight per thread (a pull
// over NVLink is bound by the bytes in flight); the peers are interleaved so that all links are busy at once.
__global__ void PullKernel(PeerTable t, char* out, size_t bytesPerRank, int nRanks, int me)
{
    const size_t nv = bytesPerRank / 16;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (int k = 0; k < nRanks; ++k) {
        const int q = (me + k) % nRanks;
        const uint4* s = reinterpret_cast<const uint4*>(t.src[q]);
        uint4* d = reinterpret_cast<uint4*>(out + (size_t)q * bytesPerRank);
        size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
        for (; i + 7 * stride < nv; i += 8 * stride) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) v[u] = s[i + u * stride];
#pragma unroll
            for (int u = 0; u < 8; ++u) d[i + u * stride] = v[u];
        }
        for (; i < nv; i += stride) d[i] = s[i];
        for (size_t b = nv * 16 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; b < bytesPerRank; b += stride)
            out[(size_t)q * bytesPerRank + b] = t.src[q][b];
    }
}

size_t TypeSize(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_FP8E4M3: case HCCL_DATA_TYPE_FP8E5M2: return 1;
        case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: return 2;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_FP32: return 4;
        case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP64: return 8;
        default: return 0;
    }
}

bool Ready() { return true; }

HcclResult Select(const HcclAlgoPluginParam* p, char name[HCCL_ALGO_PLUGIN_ALG_NAME_LEN])
{
    if (p == nullptr || p->magic != HCCL_ALGO_PLUGIN_PARAM_MAGIC || strcmp(p->opName, "AllGather") != 0) return HCCL_E_NOT_SUPPORT;
    if (p->rankNum < 2 || p->rankNum > kMaxRanks || TypeSize(p->dataType) == 0 || ((uintptr_t)p->sendBuf & 15u) != 0) return HCCL_E_NOT_SUPPORT;
    void* peer = nullptr;       // a send buffer outside symmetric memory has no peer mapping: leave the call to the library
    if (HcclCommSymWinGet(p->comm, p->sendBuf, (p->rank + 1) % p->rankNum, &peer) != HCCL_SUCCESS) return HCCL_E_NOT_SUPPORT;
    snprintf(name, HCCL_ALGO_PLUGIN_ALG_NAME_LEN, "CustomAllGatherPull");
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
    const size_t bytes = (size_t)p->count * TypeSize(p->dataType);
    cudaStream_t stream = (cudaStream_t)p->stream;
    // every rank's send buffer is final once all ranks have reached this point of their streams ...
    HcclResult r = HcclBarrier(p->comm, p->stream);
    if (r != HCCL_SUCCESS) return r;
    const int blocks = (int)((bytes / 16 + 256 * 8 - 1) / (256 * 8)) < 1 ? 1 : ((bytes / 16 + 2047) / 2048 > 128 ? 128 : (int)((bytes / 16 + 2047) / 2048));
    PullKernel<<<blocks, 256, 0, stream>>>(t, (char*)p->recvBuf, bytes, (int)p->rankNum, (int)p->rank);
    if (cudaGetLastError() != cudaSuccess) return HCCL_E_RUNTIME;
    // ... and may be overwritten again only after every rank has finished reading it
    return HcclBarrier(p->comm, p->stream);
}

HcclAlgoPluginTable g_table = {HCCL_PLUGIN_API_VERSION, HCCL_ALGO_PLUGIN_TABLE_MAGIC, sizeof(HcclAlgoPluginTable), Ready, Select, Execute};

}  // namespace

extern "C" const HcclAlgoPluginTable* GetHcclAlgoPlugin(void) { return &g_table; }
