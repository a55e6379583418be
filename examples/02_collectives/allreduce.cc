// AllReduce with one thread per GPU and root-info initialisation (the CUDA
// counterpart of HCCL's examples/02_collectives/01_allreduce/main.cc).
//
// Build (from the repository root, after `python hccl_b200/build.py`):
//   nvcc -std=c++17 -Icsrc/include examples/02_collectives/allreduce.cc -Lhccl_b200/lib -lhccl_b200 \
//        -Xlinker -rpath=$PWD/hccl_b200/lib -o allreduce_example
// Run: ./allreduce_example [nDevices]
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include "hccl/hccl.h"

#define CHECK_HCCL(x) do { HcclResult r_ = (x); if (r_ != HCCL_SUCCESS) { fprintf(stderr, "%s failed: %s\n", #x, HcclGetErrorString(r_)); exit(1); } } while (0)
#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_)); exit(1); } } while (0)

int main(int argc, char** argv)
{
    int nDev = 0;
    CHECK_CUDA(cudaGetDeviceCount(&nDev));
    if (argc > 1) nDev = atoi(argv[1]);
    const uint64_t count = 1 << 20;
    HcclRootInfo root;
    CHECK_HCCL(HcclGetRootInfo(&root));
    std::vector<std::thread> threads;
    for (int dev = 0; dev < nDev; ++dev) {
        threads.emplace_back([&, dev] {
            CHECK_CUDA(cudaSetDevice(dev));
            HcclComm comm;
            CHECK_HCCL(HcclCommInitRootInfo((uint32_t)nDev, &root, (uint32_t)dev, &comm));
            cudaStream_t stream;
            CHECK_CUDA(cudaStreamCreate(&stream));
            std::vector<float> host(count, (float)(dev + 1));
            float *send, *recv;
            CHECK_CUDA(cudaMalloc(&send, count * sizeof(float)));
            CHECK_CUDA(cudaMalloc(&recv, count * sizeof(float)));
            CHECK_CUDA(cudaMemcpy(send, host.data(), count * sizeof(float), cudaMemcpyHostToDevice));
            CHECK_HCCL(HcclAllReduce(send, recv, count, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, comm, stream));
            CHECK_CUDA(cudaStreamSynchronize(stream));
            CHECK_CUDA(cudaMemcpy(host.data(), recv, count * sizeof(float), cudaMemcpyDeviceToHost));
            const float want = nDev * (nDev + 1) / 2.0f;
            printf("rank %d: recv[0] = %.1f (expected %.1f) %s\n", dev, host[0], want, host[0] == want ? "ok" : "MISMATCH");
            HcclResult async;
            CHECK_HCCL(HcclCommGetAsyncError(comm, &async));
            if (async != HCCL_SUCCESS) fprintf(stderr, "rank %d: asynchronous error %s\n", dev, HcclGetErrorString(async));
            cudaFree(send);
            cudaFree(recv);
            cudaStreamDestroy(stream);
            CHECK_HCCL(HcclCommDestroy(comm));
        });
    }
    for (auto& t : threads) t.join();
    return 0;
}
