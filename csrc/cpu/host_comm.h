// Host engine: communicators whose ranks are host threads and whose buffers are
// host memory.  It runs the engine-agnostic algorithm templates (ring, RHD,
// NHR, mesh one/two-shot, pairwise ...) on real memory and can record every
// primitive into a trace that the verifier checks for deadlocks, races and
// semantics - the role of the reference's ST "algorithm analyzer"
// (test/st/algorithm: N ranks as N host threads in one process, HCOMM replaced
// by stubs that append TaskStubs, then Checker::DoGenAndCheckGraph,
// hccl_verifier/checker.cc:61-104).  Unlike the reference's analyzer, which is
// symbolic only, data really moves, so numeric results can be compared with an
// fp64 oracle.
#pragma once
#include "hccl/hccl_types.h"

namespace hccl {

class CommImpl;
struct OpParam;
class HostRank;   // per-rank handle into a HostWorld

// Creates `nRanks` host communicators over the topology literal `topoJson`
// ("[[[0,1,2,3],[4,5,6,7]]]" = one pod, two servers of four; empty = one server).
HcclResult HostWorldCreate(uint32_t nRanks, const char* topoJson, const HcclCommConfig* cfg, CommImpl** comms);
void HostRankRelease(HostRank* r);
HcclResult HostExecOp(CommImpl* comm, OpParam& p);

}  // namespace hccl
