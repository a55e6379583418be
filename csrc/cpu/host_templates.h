// Shared vocabulary of the host engine's algorithm templates and executors.
//
// A template runs one algorithm on one group of ranks over a working buffer W
// that every member holds at the same place (its OUTPUT buffer or a scratch
// region); an executor composes templates over the levels of a hierarchy.
// host_templates.cc defines the templates and the Sole / Sequence / Parallel /
// OrderPreserved executors, host_executors.cc the Concurrent, Pipeline,
// hierarchical AlltoAll, Bruck and tree-interpreting executors.
#pragma once
#include <cstdint>
#include <vector>
#include "../topo/topo.h"
#include "host_world.h"

namespace hccl {
namespace hosttpl {

enum Notify : uint32_t { N_READY = 0, N_DATA = 1, N_DONE = 2, N_ACK = 3, N_LEVEL = 4, N_P2P_DATA = 5, N_P2P_ACK = 6, N_AUX = 7 };

struct Group {
    std::vector<uint32_t> ranks;   // world ranks, in group order
    uint32_t me;                   // my index in `ranks`
    uint32_t size() const { return (uint32_t)ranks.size(); }
    uint32_t world(uint32_t idx) const { return ranks[idx]; }
};

// Working-buffer descriptor: where W lives on every rank (same kind and offset everywhere) and which byte range
// [base, base + bytes) of it the template works on; slices are cut in elements of `es` bytes.
struct Work {
    BufKind buf;
    uint64_t base;      // byte offset of the region inside the buffer
    uint64_t count;     // elements in the region
    uint32_t es;
    // Variable slices (the V operators): slice i of a flat group is [vBegin[i], vBegin[i] + vCount[i]) in elements
    // instead of an equal share of `count`.  Null for the regular operators.
    const uint64_t* vBegin = nullptr;
    const uint64_t* vCount = nullptr;
    Mem At(uint32_t worldRank, uint64_t elemOff) const { return Mem{worldRank, buf, base + elemOff * es}; }
};

struct Ctx {
    HostWorld& w;
    HostPrims& x;
    uint32_t q;          // queue for the recorded tasks
    uint64_t scratchOff; // start of the scratch area this template may use (bytes)
    uint64_t scratchLen;
};

enum class Fam { MESH, RING, NHR, RHD };

void Slice(const Work& wk, uint32_t parts, uint32_t i, uint64_t* b, uint64_t* e);
// The region of `wk` that slice `idx` of `parts` covers, as a Work of its own.
Work SubWork(const Work& wk, uint32_t parts, uint32_t idx);

// Templates.  ReduceScatter: afterwards member i holds the reduced slice i of W.  AllGather: member i enters with
// slice i valid, all leave with every slice.  AllReduce: both, or the one-shot mesh with the fixed fold order.
void MeshReduceScatter(Ctx& c, const Group& g, const Work& wk);
void MeshAllGather(Ctx& c, const Group& g, const Work& wk);
void MeshOneShotAllReduce(Ctx& c, const Group& g, const Work& wk);
void RingReduceScatter(Ctx& c, const Group& g, const Work& wk);
void RingAllGather(Ctx& c, const Group& g, const Work& wk);
void NhrReduceScatter(Ctx& c, const Group& g, const Work& wk);
void NhrAllGather(Ctx& c, const Group& g, const Work& wk);
void RhdReduceScatter(Ctx& c, const Group& g, const Work& wk, bool skipPost);
void RhdAllGather(Ctx& c, const Group& g, const Work& wk, bool skipPre);
void ReduceScatterBy(Fam f, Ctx& c, const Group& g, const Work& wk);
void AllGatherBy(Fam f, Ctx& c, const Group& g, const Work& wk);
void AllReduceBy(Fam f, Ctx& c, const Group& g, const Work& wk);

Group WholeGroup(HostWorld& w, uint32_t rank);
bool LevelGroup(const AlgHierarchy& h, uint32_t level, uint32_t rank, Group* out);
// Sequence AllReduce over the levels of `h` on region wk: ReduceScatter down the levels, AllReduce at the top,
// AllGather back up; fam[l] names the template family of level l.
void SequenceAllReduce(Ctx& c, const AlgHierarchy& h, uint32_t rank, const Work& wk, const std::vector<Fam>& fam);

}  // namespace hosttpl

// Executors of host_executors.cc.  Returns HCCL_E_NOT_SUPPORT when `alg` is not one of them.
HcclResult RunHostExecutorExt(HostWorld& w, uint32_t rank, int alg, const OpParam& p);

}  // namespace hccl
