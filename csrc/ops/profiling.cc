#include "profiling.h"
#include "param_check.h"
#include <nvtx3/nvToolsExt.h>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>

namespace hccl {
namespace {
struct Pending { ProfRecord rec; cudaEvent_t e0, e1; };
struct ProfState {
    int level = 0;
    std::mutex mu;
    std::deque<ProfRecord> done;
    std::deque<Pending> pending;
    uint64_t seq = 0;
    ProfState() { if (const char* e = getenv("HCCL_PROFILING")) level = atoi(e); }
};
ProfState& S() { static ProfState s; return s; }
constexpr size_t kRing = 4096;

void Drain(ProfState& s, bool wait)
{
    while (!s.pending.empty()) {
        Pending& p = s.pending.front();
        cudaError_t q = wait ? cudaEventSynchronize(p.e1) : cudaEventQuery(p.e1);
        if (q != cudaSuccess) { cudaGetLastError(); if (!wait) break; }
        float ms = -1.f;
        if (q == cudaSuccess && cudaEventElapsedTime(&ms, p.e0, p.e1) == cudaSuccess) p.rec.deviceUs = ms * 1000.0;
        cudaEventDestroy(p.e0);
        cudaEventDestroy(p.e1);
        if (s.done.size() >= kRing) s.done.pop_front();
        s.done.push_back(p.rec);
        s.pending.pop_front();
    }
}
}  // namespace

int ProfilingLevel() { return S().level; }
void SetProfilingLevel(int level) { S().level = level; }
std::vector<ProfRecord> ProfilingSnapshot()
{
    ProfState& s = S();
    std::lock_guard<std::mutex> lk(s.mu);
    Drain(s, true);
    return std::vector<ProfRecord>(s.done.begin(), s.done.end());
}
void ProfilingClear()
{
    ProfState& s = S();
    std::lock_guard<std::mutex> lk(s.mu);
    Drain(s, true);
    s.done.clear();
}

// NVTX range per operator (visible in Nsight Systems / Compute timelines): on with HCCL_NVTX=1.  The header-only
// NVTX v3 does nothing until a tool injects itself, so an enabled range costs a few nanoseconds without a profiler.
static bool NvtxEnabled()
{
    static const bool on = [] { const char* e = getenv("HCCL_NVTX"); return e != nullptr && e[0] == '1'; }();
    return on;
}

ProfilingScope::ProfilingScope(CommImpl* c, const OpParam& p, const char* alg, uint64_t bytes)
{
    if (NvtxEnabled()) {
        char label[160];
        snprintf(label, sizeof(label), "Hccl%s %s %llu B", CmdName(p.op), alg, (unsigned long long)bytes);
        nvtxRangePushA(label);
        nvtx_ = true;
    }
    ProfState& s = S();
    if (s.level <= 0) return;
    on_ = true;
    rec_.op = (uint32_t)p.op; rec_.dtype = (uint32_t)p.dtype; rec_.rank = (uint32_t)c->rank; rec_.rankSize = (uint32_t)c->nRanks;
    rec_.root = p.root; rec_.count = p.count; rec_.bytes = bytes; rec_.deviceUs = -1;
    snprintf(rec_.alg, sizeof(rec_.alg), "%s", alg);
    snprintf(rec_.comm, sizeof(rec_.comm), "%s", c->name.c_str());
    snprintf(rec_.tag, sizeof(rec_.tag), "%s", p.tag.c_str());
    stream_ = p.stream;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    // events with timing cannot be recorded into a capturing stream
    if (s.level >= 2 && !c->hostComm && cudaStreamIsCapturing(stream_, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone &&
        cudaEventCreate(&ev0_) == cudaSuccess && cudaEventCreate(&ev1_) == cudaSuccess)
        cudaEventRecord(ev0_, stream_);
}

ProfilingScope::~ProfilingScope()
{
    if (nvtx_) nvtxRangePop();
    if (!on_) return;
    ProfState& s = S();
    rec_.hostSubmitUs = hostUs_;
    std::lock_guard<std::mutex> lk(s.mu);
    rec_.seq = ++s.seq;
    if (ev0_ && ev1_) {
        cudaEventRecord(ev1_, stream_);
        s.pending.push_back({rec_, ev0_, ev1_});
        Drain(s, s.pending.size() > 1024);
    } else {
        if (s.done.size() >= kRing) s.done.pop_front();
        s.done.push_back(rec_);
    }
}

}  // namespace hccl
