// Ring exchange with HcclBatchSendRecv: every rank sends to its right neighbour and receives from its left one in
// one call (the CUDA counterpart of HCCL's examples/01_point_to_point/02_batch_send_recv_ring).
// Build / run as examples/02_collectives/allreduce.cc.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include "hccl/hccl.h"

#define CHECK_HCCL(x) do { HcclResult r_ = (x); if (r_ != HCCL_SUCCESS) { fprintf(stderr, "%s failed: %s\n", #x, HcclGetErrorString(r_)); exit(1); } } while (0)

int main(int argc, char** argv)
{
    int nDev = 0;
    cudaGetDeviceCount(&nDev);
    if (argc > 1) nDev = atoi(argv[1]);
    const uint64_t count = 4096;
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
            int32_t *send, *recv;
            cudaMalloc(&send, count * 4);
            cudaMalloc(&recv, count * 4);
            std::vector<int32_t> host(count, dev);
            cudaMemcpy(send, host.data(), count * 4, cudaMemcpyHostToDevice);
            HcclSendRecvItem items[2];
            items[0] = {HCCL_SEND, send, count, HCCL_DATA_TYPE_INT32, (uint32_t)((dev + 1) % nDev)};
            items[1] = {HCCL_RECV, recv, count, HCCL_DATA_TYPE_INT32, (uint32_t)((dev + nDev - 1) % nDev)};
            CHECK_HCCL(HcclBatchSendRecv(items, 2, comm, stream));
            cudaStreamSynchronize(stream);
            cudaMemcpy(host.data(), recv, count * 4, cudaMemcpyDeviceToHost);
            printf("rank %d received from rank %d: %s\n", dev, host[0], host[0] == (dev + nDev - 1) % nDev ? "ok" : "MISMATCH");
            cudaFree(send);
            cudaFree(recv);
            cudaStreamDestroy(stream);
            CHECK_HCCL(HcclCommDestroy(comm));
        });
    }
    for (auto& t : threads) t.join();
    return 0;
}
