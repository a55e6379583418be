// Per-operator profiling records.
//
// Reference: HcomProInfo (alg_param.h:880-898: dtype, cmd, count, rank size,
// rank, block dim, begin time, root, tag, comm, algorithm) reported at
// HcclExecOp entry / exit (op_common.cc:1265, :1440) through msprof hooks.
// Here: a ring of records per process, filled when HCCL_PROFILING=1 (host
// submit time always; device time from CUDA events recorded around the op on
// its stream when HCCL_PROFILING=2), readable through HcclProfilingDump.
// HCCL_NVTX=1 additionally wraps every operator in an NVTX range.
#pragma once
#include <cstdint>
#include <string>
#include <vector>
#include "op_common.h"

namespace hccl {

struct ProfRecord {
    uint64_t seq;
    uint32_t op, dtype, rank, rankSize, root;
    uint64_t count, bytes;
    double hostSubmitUs;
    double deviceUs;      // < 0: not measured
    char alg[64];
    char comm[64];
    char tag[64];
};

int ProfilingLevel();                 // 0 off, 1 host timing, 2 + device events
void SetProfilingLevel(int level);
std::vector<ProfRecord> ProfilingSnapshot();
void ProfilingClear();

class ProfilingScope {
public:
    ProfilingScope(CommImpl* c, const OpParam& p, const char* alg, uint64_t bytes);
    ~ProfilingScope();
    void SetHostUs(double us) { hostUs_ = us; }
private:
    bool on_ = false;
    bool nvtx_ = false;
    ProfRecord rec_{};
    double hostUs_ = 0;
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    cudaStream_t stream_ = nullptr;
};

}  // namespace hccl
