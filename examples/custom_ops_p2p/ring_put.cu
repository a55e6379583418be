// A user-written point-to-point transfer built from the public programming model only (the counterpart of HCCL's
// examples/04_custom_ops_p2p): every rank PUTS its block into its right neighbour's buffer with an own kernel that
// stores through the neighbour's mapping of a symmetric allocation.
//
//   HcclMemAlloc          one buffer per rank, mapped on every peer
//   HcclCommSymWinGet     the neighbour's mapping of my buffer's twin
//   HcclBarrier           "the destination may be written" before the put, "the data has landed" after it
//
// Threads are the ranks (one GPU each).  Build, from the repository root after `python hccl_b200/build.py`:
//   nvcc -std=c++17 -gencode arch=compute_100a,code=sm_100a -Icsrc/include examples/custom_ops_p2p/ring_put.cu \
//        -Lhccl_b200/lib -lhccl_b200 -Xlinker -rpath=$PWD/hccl_b200/lib -o ring_put
// Run: ./ring_put [nGpus]
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include "hccl/hccl.h"
#include "hccl/hccl_comm.h"

#define CHECK_HCCL(x) do { HcclResult r_ = (x); if (r_ != HCCL_SUCCESS) { fprintf(stderr, "%s failed: %s\n", #x, HcclGetErrorString(r_)); exit(1); } } while (0)

// dst lives on the neighbour GPU; sixteen-byte stores, four in flight per thread.
__global__ void PutKernel(uint4* dst, const uint4* src, size_t nVec)
{
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nVec; i += 4 * stride) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = src[i + u * stride];
#pragma unroll
        for (int u = 0; u < 4; ++u) dst[i + u * stride] = v[u];
    }
    for (; i < nVec; i += stride) dst[i] = src[i];
}

int main(int argc, char** argv)
{
    int nDev = 0;
    cudaGetDeviceCount(&nDev);
    if (argc > 1) nDev = atoi(argv[1]);
    if (nDev < 2) { printf("needs at least two GPUs\n"); return 0; }
    const size_t count = 1 << 20;                       // int32 elements per rank
    HcclRootInfo root;
    CHECK_HCCL(HcclGetRootInfo(&root));
    std::vector<std::thread> threads;
    for (int dev = 0; dev < nDev; ++dev) {
        threads.emplace_back([&, dev] {
            cudaSetDevice(dev);
            HcclComm comm;
            CHECK_HCCL(HcclCommInitRootInfo((uint32_t)nDev, &root, (uint32_t)dev, &comm));
            cudaStream_t stream;
            cudaStreamCreate(&stream);
            // inbox: symmetric (collective allocation), so the left neighbour can store into it
            void* inbox = nullptr;
            CHECK_HCCL(HcclMemAlloc(comm, count * 4, &inbox));
            int32_t* outbox = nullptr;
            cudaMalloc(&outbox, count * 4);
            std::vector<int32_t> host(count, dev);
            cudaMemcpy(outbox, host.data(), count * 4, cudaMemcpyHostToDevice);
            const uint32_t right = (uint32_t)((dev + 1) % nDev);
            void* rightInbox = nullptr;                 // the right neighbour's inbox as mapped on this GPU
            CHECK_HCCL(HcclCommSymWinGet(comm, inbox, right, &rightInbox));
            CHECK_HCCL(HcclBarrier(comm, stream));      // every inbox exists and may be written
            PutKernel<<<64, 256, 0, stream>>>((uint4*)rightInbox, (const uint4*)outbox, count * 4 / 16);
            CHECK_HCCL(HcclBarrier(comm, stream));      // every put has landed
            cudaStreamSynchronize(stream);
            cudaMemcpy(host.data(), inbox, count * 4, cudaMemcpyDeviceToHost);
            const int left = (dev + nDev - 1) % nDev;
            printf("rank %d holds the block of rank %d: %s\n", dev, host[0], host[0] == left && host[count - 1] == left ? "ok" : "MISMATCH");
            cudaFree(outbox);
            CHECK_HCCL(HcclMemFree(comm, inbox));
            cudaStreamDestroy(stream);
            CHECK_HCCL(HcclCommDestroy(comm));
        });
    }
    for (auto& t : threads) t.join();
    return 0;
}
