// Sizing the communication nodes of a graph before any communicator exists: what a graph builder does when it plans
// streams and workspace ahead of time (the counterpart of HCCL's HcclCreateOpParamGraphMode / HcclSetOpParamGraphMode* /
// HcclCalcOpRes*GraphMode family).  Needs no GPU: the answers come from the selector and the cost model on a
// described box.
//
// Build (from the repository root, after `python hccl_b200/build.py`):
//   nvcc -std=c++17 -Icsrc/include examples/04_graph_mode/node_resources.cc -Lhccl_b200/lib -lhccl_b200 \
//        -Xlinker -rpath=$PWD/hccl_b200/lib -o node_resources
// Run: ./node_resources [nRanks] [slabMiB]
#include <cstdio>
#include <cstdlib>
#include "hccl/hccl_graph_mode.h"

#define CHECK_HCCL(x) do { HcclResult r_ = (x); if (r_ != HCCL_SUCCESS) { fprintf(stderr, "%s failed: %s\n", #x, HcclGetErrorString(r_)); exit(1); } } while (0)

struct Node { const char* op; uint64_t count; HcclDataType type; int registered; };

int main(int argc, char** argv)
{
    const uint32_t nRanks = argc > 1 ? (uint32_t)atoi(argv[1]) : 8;
    const uint64_t slab = (argc > 2 ? (uint64_t)atoi(argv[2]) : 256) << 20;
    // the communication nodes of one tensor-parallel decoder layer and of a data-parallel gradient step
    const Node nodes[] = {
        {"HcomAllGather", 4096ull * 8192 / nRanks, HCCL_DATA_TYPE_BFP16, 1},       // sequence shard -> full activations
        {"HcomReduceScatter", 4096ull * 8192 / nRanks, HCCL_DATA_TYPE_BFP16, 1},   // partial sums -> sequence shard
        {"HcomAllReduce", 8192, HCCL_DATA_TYPE_FP32, 0},                           // a replicated norm weight's gradient
        {"HcomAllReduce", 512ull << 20, HCCL_DATA_TYPE_BFP16, 0},                  // a 1 GiB gradient bucket in ordinary memory
        {"HcomAlltoAll", (64ull << 20) / nRanks, HCCL_DATA_TYPE_BFP16, 1},         // expert dispatch
        {"HcomBroadcast", 1ull << 20, HCCL_DATA_TYPE_FP32, 0},                     // parameters at start-up
    };
    printf("%u GPUs behind one switch, %llu MiB slab\n", nRanks, (unsigned long long)(slab >> 20));
    printf("%-20s %14s %6s %11s | %-36s %9s %8s %6s\n", "node", "count", "type", "buffers", "algorithm", "slab KiB", "launches", "grid");
    for (const Node& n : nodes) {
        HcclOpParamGraphMode* p = nullptr;
        CHECK_HCCL(HcclCreateOpParamGraphMode(&p));
        CHECK_HCCL(HcclSetOpParamGraphModeOpType(p, n.op));
        CHECK_HCCL(HcclSetOpParamGraphModeDataCount(p, n.count));
        CHECK_HCCL(HcclSetOpParamGraphModeDataType(p, n.type));
        CHECK_HCCL(HcclSetOpParamGraphModeRankSize(p, nRanks));
        CHECK_HCCL(HcclSetOpParamGraphModeHCCLBufferSize(p, slab));
        CHECK_HCCL(HcclSetOpParamGraphModeRegistered(p, n.registered, /*switchReduces=*/1));
        uint64_t mem = 0;
        uint32_t streams = 0, launches = 0, blocks = 0;
        char alg[128];
        CHECK_HCCL(HcclCalcOpResOpParamGraphMode(p, &mem, &streams, &launches, &blocks, alg));
        printf("%-20s %14llu %6s %11s | %-36s %9llu %8u %6u\n", n.op, (unsigned long long)n.count, n.type == HCCL_DATA_TYPE_BFP16 ? "bf16" : "fp32",
               n.registered ? "symmetric" : "ordinary", alg, (unsigned long long)(mem >> 10), launches, blocks);
        CHECK_HCCL(HcclDestroyOpParamGraphMode(p));
    }
    return 0;
}
