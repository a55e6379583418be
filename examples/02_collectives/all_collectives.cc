// The ten collectives beside AllReduce, one thread per GPU, each checked on the host: Broadcast, AllGather,
// ReduceScatter, Reduce, AlltoAll, AlltoAllV, AlltoAllVC, Scatter, AllGatherV, ReduceScatterV (the CUDA counterpart
// of HCCL's examples/02_collectives/02_broadcast .. 11_reduce_scatterv).
//
// Build (from the repository root, after `python hccl_b200/build.py`):
//   nvcc -std=c++17 -Icsrc/include examples/02_collectives/all_collectives.cc -Lhccl_b200/lib -lhccl_b200 \
//        -Xlinker -rpath=$PWD/hccl_b200/lib -o all_collectives_example
// Run: ./all_collectives_example [nDevices]
//
// Rank r fills element i of a block meant for / coming from rank q with the value 1000*r + q + i*1e-3, so that every
// result has a closed form.
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <thread>
#include <vector>
#include "hccl/hccl.h"

#define CHECK_HCCL(x) do { HcclResult r_ = (x); if (r_ != HCCL_SUCCESS) { fprintf(stderr, "%s failed: %s\n", #x, HcclGetErrorString(r_)); exit(1); } } while (0)
#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_)); exit(1); } } while (0)

namespace {

struct Rank {
    int me, n;
    HcclComm comm;
    cudaStream_t stream;
    float *dSend, *dRecv;
    size_t cap;      // elements per device buffer
    int failures = 0;

    void Upload(const std::vector<float>& h) { CHECK_CUDA(cudaMemcpy(dSend, h.data(), h.size() * sizeof(float), cudaMemcpyHostToDevice)); }
    std::vector<float> Download(size_t count, bool fromSend = false)
    {
        CHECK_CUDA(cudaStreamSynchronize(stream));
        std::vector<float> h(count);
        CHECK_CUDA(cudaMemcpy(h.data(), fromSend ? dSend : dRecv, count * sizeof(float), cudaMemcpyDeviceToHost));
        return h;
    }
    void Expect(const char* what, bool ok)
    {
        if (!ok) ++failures;
        if (me == 0 || !ok) printf("rank %d: %-16s %s\n", me, what, ok ? "ok" : "MISMATCH");
    }
};

float Val(int from, int to, size_t i) { return 1000.0f * from + to + (float)i * 1e-3f; }
bool Near(float a, float b) { return std::fabs(a - b) <= 1e-3f * std::fabs(b) + 1e-3f; }

void Run(Rank& r)
{
    const int n = r.n, me = r.me;
    const size_t per = 4096;                       // elements per block
    // ---- Broadcast from the last rank
    {
        std::vector<float> h(per);
        for (size_t i = 0; i < per; ++i) h[i] = Val(me, 0, i);
        r.Upload(h);
        CHECK_HCCL(HcclBroadcast(r.dSend, per, HCCL_DATA_TYPE_FP32, (uint32_t)(n - 1), r.comm, r.stream));
        auto out = r.Download(per, true);
        bool ok = true;
        for (size_t i = 0; i < per; ++i) ok = ok && out[i] == Val(n - 1, 0, i);
        r.Expect("Broadcast", ok);
    }
    // ---- AllGather
    {
        std::vector<float> h(per);
        for (size_t i = 0; i < per; ++i) h[i] = Val(me, 0, i);
        r.Upload(h);
        CHECK_HCCL(HcclAllGather(r.dSend, r.dRecv, per, HCCL_DATA_TYPE_FP32, r.comm, r.stream));
        auto out = r.Download(per * n);
        bool ok = true;
        for (int q = 0; q < n; ++q)
            for (size_t i = 0; i < per; ++i) ok = ok && out[q * per + i] == Val(q, 0, i);
        r.Expect("AllGather", ok);
    }
    // ---- ReduceScatter (sum) and Reduce (sum, root 0)
    {
        std::vector<float> h(per * n);
        for (int q = 0; q < n; ++q)
            for (size_t i = 0; i < per; ++i) h[q * per + i] = Val(me, q, i);
        r.Upload(h);
        CHECK_HCCL(HcclReduceScatter(r.dSend, r.dRecv, per, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, r.comm, r.stream));
        auto out = r.Download(per);
        bool ok = true;
        for (size_t i = 0; i < per; ++i) {
            float want = 0;
            for (int q = 0; q < n; ++q) want += Val(q, me, i);
            ok = ok && Near(out[i], want);
        }
        r.Expect("ReduceScatter", ok);
        CHECK_HCCL(HcclReduce(r.dSend, r.dRecv, per, HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, 0, r.comm, r.stream));
        out = r.Download(per);
        ok = true;
        if (me == 0)
            for (size_t i = 0; i < per; ++i) {
                float want = 0;
                for (int q = 0; q < n; ++q) want += Val(q, 0, i);
                ok = ok && Near(out[i], want);
            }
        r.Expect("Reduce", ok);
    }
    // ---- AlltoAll
    {
        std::vector<float> h(per * n);
        for (int q = 0; q < n; ++q)
            for (size_t i = 0; i < per; ++i) h[q * per + i] = Val(me, q, i);
        r.Upload(h);
        CHECK_HCCL(HcclAlltoAll(r.dSend, per, HCCL_DATA_TYPE_FP32, r.dRecv, per, HCCL_DATA_TYPE_FP32, r.comm, r.stream));
        auto out = r.Download(per * n);
        bool ok = true;
        for (int q = 0; q < n; ++q)
            for (size_t i = 0; i < per; ++i) ok = ok && out[q * per + i] == Val(q, me, i);
        r.Expect("AlltoAll", ok);
    }
    // ---- AlltoAllV and AlltoAllVC: rank s sends (s + d + 1) * 100 elements to rank d
    {
        auto cnt = [](int s, int d) { return (uint64_t)(s + d + 1) * 100; };
        std::vector<uint64_t> sc(n), sd(n), rc(n), rd(n), matrix((size_t)n * n);
        uint64_t so = 0, ro = 0;
        for (int q = 0; q < n; ++q) {
            sc[q] = cnt(me, q); sd[q] = so; so += sc[q];
            rc[q] = cnt(q, me); rd[q] = ro; ro += rc[q];
            for (int d = 0; d < n; ++d) matrix[(size_t)q * n + d] = cnt(q, d);
        }
        std::vector<float> h(so);
        for (int q = 0; q < n; ++q)
            for (uint64_t i = 0; i < sc[q]; ++i) h[sd[q] + i] = Val(me, q, i);
        for (int variant = 0; variant < 2; ++variant) {
            r.Upload(h);
            CHECK_CUDA(cudaMemsetAsync(r.dRecv, 0, ro * sizeof(float), r.stream));
            if (variant == 0)
                CHECK_HCCL(HcclAlltoAllV(r.dSend, sc.data(), sd.data(), HCCL_DATA_TYPE_FP32, r.dRecv, rc.data(), rd.data(), HCCL_DATA_TYPE_FP32,
                                         r.comm, r.stream));
            else
                CHECK_HCCL(HcclAlltoAllVC(r.dSend, matrix.data(), HCCL_DATA_TYPE_FP32, r.dRecv, HCCL_DATA_TYPE_FP32, r.comm, r.stream));
            auto out = r.Download(ro);
            bool ok = true;
            for (int q = 0; q < n; ++q)
                for (uint64_t i = 0; i < rc[q]; ++i) ok = ok && out[rd[q] + i] == Val(q, me, i);
            r.Expect(variant == 0 ? "AlltoAllV" : "AlltoAllVC", ok);
        }
    }
    // ---- Scatter from rank 0
    {
        std::vector<float> h(per * n);
        for (int q = 0; q < n; ++q)
            for (size_t i = 0; i < per; ++i) h[q * per + i] = Val(me, q, i);
        r.Upload(h);
        CHECK_HCCL(HcclScatter(r.dSend, r.dRecv, per, HCCL_DATA_TYPE_FP32, 0, r.comm, r.stream));
        auto out = r.Download(per);
        bool ok = true;
        for (size_t i = 0; i < per; ++i) ok = ok && out[i] == Val(0, me, i);
        r.Expect("Scatter", ok);
    }
    // ---- AllGatherV and ReduceScatterV: rank q owns (q + 1) * 300 elements
    {
        std::vector<uint64_t> counts(n), displs(n);
        uint64_t total = 0;
        for (int q = 0; q < n; ++q) { counts[q] = (uint64_t)(q + 1) * 300; displs[q] = total; total += counts[q]; }
        std::vector<float> h(counts[me]);
        for (uint64_t i = 0; i < counts[me]; ++i) h[i] = Val(me, 0, i);
        r.Upload(h);
        CHECK_HCCL(HcclAllGatherV(r.dSend, counts[me], r.dRecv, counts.data(), displs.data(), HCCL_DATA_TYPE_FP32, r.comm, r.stream));
        auto out = r.Download(total);
        bool ok = true;
        for (int q = 0; q < n; ++q)
            for (uint64_t i = 0; i < counts[q]; ++i) ok = ok && out[displs[q] + i] == Val(q, 0, i);
        r.Expect("AllGatherV", ok);

        std::vector<float> full(total);
        for (int q = 0; q < n; ++q)
            for (uint64_t i = 0; i < counts[q]; ++i) full[displs[q] + i] = Val(me, q, i);
        r.Upload(full);
        CHECK_HCCL(HcclReduceScatterV(r.dSend, counts.data(), displs.data(), r.dRecv, counts[me], HCCL_DATA_TYPE_FP32, HCCL_REDUCE_SUM, r.comm,
                                      r.stream));
        out = r.Download(counts[me]);
        ok = true;
        for (uint64_t i = 0; i < counts[me]; ++i) {
            float want = 0;
            for (int q = 0; q < n; ++q) want += Val(q, me, i);
            ok = ok && Near(out[i], want);
        }
        r.Expect("ReduceScatterV", ok);
    }
    CHECK_HCCL(HcclBarrier(r.comm, r.stream));
    CHECK_CUDA(cudaStreamSynchronize(r.stream));
}

}  // namespace

int main(int argc, char** argv)
{
    int nDev = 0;
    CHECK_CUDA(cudaGetDeviceCount(&nDev));
    if (argc > 1) nDev = atoi(argv[1]);
    HcclRootInfo root;
    CHECK_HCCL(HcclGetRootInfo(&root));
    std::vector<std::thread> threads;
    std::vector<int> failures((size_t)nDev, 0);
    for (int dev = 0; dev < nDev; ++dev) {
        threads.emplace_back([&, dev] {
            CHECK_CUDA(cudaSetDevice(dev));
            Rank r;
            r.me = dev; r.n = nDev;
            CHECK_HCCL(HcclCommInitRootInfo((uint32_t)nDev, &root, (uint32_t)dev, &r.comm));
            CHECK_CUDA(cudaStreamCreate(&r.stream));
            r.cap = (size_t)4096 * nDev + (size_t)nDev * nDev * 300;
            CHECK_CUDA(cudaMalloc(&r.dSend, r.cap * sizeof(float)));
            CHECK_CUDA(cudaMalloc(&r.dRecv, r.cap * sizeof(float)));
            Run(r);
            HcclResult async;
            CHECK_HCCL(HcclCommGetAsyncError(r.comm, &async));
            if (async != HCCL_SUCCESS) { fprintf(stderr, "rank %d: asynchronous error %s\n", dev, HcclGetErrorString(async)); ++r.failures; }
            failures[(size_t)dev] = r.failures;
            cudaFree(r.dSend);
            cudaFree(r.dRecv);
            cudaStreamDestroy(r.stream);
            CHECK_HCCL(HcclCommDestroy(r.comm));
        });
    }
    for (auto& t : threads) t.join();
    int bad = 0;
    for (int f : failures) bad += f;
    printf(bad == 0 ? "all collectives ok on %d ranks\n" : "%d mismatches on %d ranks\n", bad == 0 ? nDev : bad, nDev);
    return bad == 0 ? 0 : 1;
}
