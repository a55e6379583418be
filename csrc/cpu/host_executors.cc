// Executors and templates of the host engine beyond the Sole / Sequence /
// Parallel / OrderPreserved set of host_templates.cc:
//
//   Concurrent - two templates on the same ranks over two disjoint link sets
//       (the reference pairs the mesh links with the CLOS links and costs the
//       pair with CostAggMode::MAX, executor_v2_base.h:130-141,
//       ins_v2_all_reduce_concurrent_executor.cc): the data is split by the
//       bandwidth ratio, part A runs the mesh template on queue 0 while part B
//       runs NHR on queue 1.
//   Pipeline (the reference's OmniPipe / PipeLine 2D and 3D executors,
//       ins_v2_all_reduce_omnipipe_executor.cc, coll_algo_intro/Pipeline.md):
//       the data is cut in at most five steps; step i's inter-server stage runs
//       beside step i + 1's intra-server stage, each stage on its own queue;
//       AllReduce also on three levels (server, pod, pods) in five stages.
//   Nonuniform Bruck (HCCL_ALGO "NB", scatter_nb.cc): AllGather, Broadcast and a
//       binomial-tree Scatter in ceil(log2 p) steps for any p.
//   Hierarchical AlltoAll(V/VC) (all_to_all_v/.../aicpu/hier/*): intra-server
//       stage into relays, meta table, inter-server stage.
//   Sequence forms of Broadcast, Reduce, Scatter and Barrier on two levels.
//   Mesh with a detour (the reference's Z-axis detour templates): AllGather,
//       ReduceScatter and Scatter whose pair transfers are split over two
//       channels by bandwidth.
//   Tree executor (experimental/ops/op_common/recursive_executor/*, RFC 0003):
//       one executor that interprets a tree of seq / par / rev nodes with
//       template leaves, given in HCCL_ALGO_TREE.
#include <algorithm>
#include <cstring>
#include <memory>
#include <numeric>
#include "../core/config.h"
#include "../core/log.h"
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "host_templates.h"
#include "host_tree.h"
#include "host_world.h"

namespace hccl {
using namespace hosttpl;

namespace {

uint64_t Bytes(const OpParam& p) { return p.count * DataTypeSize(p.dtype); }

// Bandwidth shares of the two link sets of a Concurrent / Parallel split.  Default: the reference's own figures for
// its mesh links (56) and CLOS links (112) (rfcs/0003-executor-template-refactor.md:724);
// HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO="a,b" overrides them.
void SplitShares(double* a, double* b)
{
    const EnvConfig& env = GetEnvConfig();
    *a = 56.0;
    *b = 112.0;
    if (env.splitRatio.size() >= 2 && env.splitRatio[0] + env.splitRatio[1] > 0) { *a = env.splitRatio[0]; *b = env.splitRatio[1]; }
}

const std::vector<uint32_t>* GroupOf(const AlgHierarchy& h, uint32_t level, uint32_t rank)
{
    for (auto& grp : h.infos[level])
        if (std::find(grp.begin(), grp.end(), rank) != grp.end()) return &grp;
    return nullptr;
}
uint32_t IndexIn(const std::vector<uint32_t>& grp, uint32_t rank) { return (uint32_t)(std::find(grp.begin(), grp.end(), rank) - grp.begin()); }

// ---------------------------------------------------------------- Nonuniform Bruck
void NbAllGather(Ctx& c, const Group& g, const Work& wk)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const uint32_t me = g.world(g.me);
    for (const BruckStep& s : BruckAllGatherSteps(p, g.me)) {
        const uint32_t to = g.world(s.sendTo), from = g.world(s.recvFrom);
        c.x.Post(from, N_READY, c.q);      // my W may be written
        c.x.Wait(to, N_READY, c.q);
        for (uint32_t k = 0; k < s.nBlocks; ++k) {
            uint64_t b, e;
            Slice(wk, p, (s.firstSendBlock + k) % p, &b, &e);
            c.x.Copy(wk.At(to, b), wk.At(me, b), (e - b) * wk.es, c.q);
        }
        c.x.Post(to, N_DATA, c.q);
        c.x.Wait(from, N_DATA, c.q);
    }
}

HcclResult NbScatter(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size();
    const uint64_t blk = Bytes(p);
    if ((uint64_t)n * blk > w.scratchBytes()) {
        HCCL_ERROR("host engine: tree Scatter stages %llu bytes, the scratch buffer has %llu (raise HCCL_BUFFSIZE)", (unsigned long long)(n * blk),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const uint32_t v = (rank + n - p.root) % n;
    x.SyncGroup(all.ranks, N_READY);
    for (const TreeScatterStep& s : BinomialScatterSteps(n, v)) {
        const uint32_t peer = (p.root + s.peer) % n;
        if (s.sends) {
            for (uint32_t k = 0; k < s.nBlocks; ++k) {
                const uint32_t rel = s.firstBlock + k, owner = (p.root + rel) % n;
                const Mem src = rank == p.root ? In(rank, (uint64_t)owner * blk) : Scratch(rank, (uint64_t)rel * blk);
                x.Copy(Scratch(peer, (uint64_t)rel * blk), src, blk);
            }
            x.Post(peer, N_DATA);
        } else if (s.receives) {
            x.Wait(peer, N_DATA);
        }
    }
    if (rank == p.root) x.Copy(Out(rank), In(rank, (uint64_t)rank * blk), blk);
    else x.Copy(Out(rank), Scratch(rank, (uint64_t)v * blk), blk);
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- Concurrent
// AllReduce on OUTPUT (already holding the rank's input): part A mesh two-shot, part B NHR.
void ConcurrentAllReduce(HostWorld& w, HostPrims& x, const Group& all, const Work& wk)
{
    double sa, sb;
    SplitShares(&sa, &sb);
    const uint64_t a = BandwidthSplit(wk.count, sa, sb, std::max<uint64_t>(1, 128 / wk.es));
    const Work A{wk.buf, wk.base, a, wk.es}, B{wk.buf, wk.base + a * wk.es, wk.count - a, wk.es};
    Ctx ca{w, x, 0, 0, 0};
    Ctx cb{w, x, 1, 0, w.scratchBytes()};
    if (A.count) AllReduceBy(Fam::MESH, ca, all, A);
    if (B.count) AllReduceBy(Fam::NHR, cb, all, B);
}

// ReduceScatter: W_A / W_B are the two parts of every rank's blocks, laid out part by part in the upper half of scratch.
void ConcurrentReduceScatter(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    double sa, sb;
    SplitShares(&sa, &sb);
    const uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es)), b = p.count - a;
    const uint64_t wOff = w.scratchBytes() / 2;
    const Work A{BufKind::SCRATCH, wOff, a * n, es}, B{BufKind::SCRATCH, wOff + a * n * es, b * n, es};
    for (uint32_t j = 0; j < n; ++j) {
        if (a) x.Copy(A.At(rank, (uint64_t)j * a), In(rank, (uint64_t)j * p.count * es), a * es);
        if (b) x.Copy(B.At(rank, (uint64_t)j * b), In(rank, ((uint64_t)j * p.count + a) * es), b * es, 1);
    }
    Ctx ca{w, x, 0, 0, 0};
    Ctx cb{w, x, 1, 0, w.scratchBytes() / 2};
    if (a) { MeshReduceScatter(ca, all, A); x.Copy(Out(rank), A.At(rank, (uint64_t)rank * a), a * es); }
    if (b) { NhrReduceScatter(cb, all, B); x.Copy(Out(rank, a * es), B.At(rank, (uint64_t)rank * b), b * es, 1); }
    x.SyncGroup(all.ranks, N_LEVEL);     // nobody reuses its scratch while a peer may still read it
}

// AllGather: part A of every block is pulled straight from the owner's INPUT over the mesh; part B is gathered by NHR
// in scratch and copied out.
void ConcurrentAllGather(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    double sa, sb;
    SplitShares(&sa, &sb);
    uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es));
    if ((p.count - a) * n * es > w.scratchBytes()) a = p.count;      // part B has to fit the staging buffer
    const uint64_t b = p.count - a;
    x.SyncGroup(all.ranks, N_READY);
    for (uint32_t k = 0; k < n && a; ++k) {
        const uint32_t j = (rank + k) % n;
        x.Copy(Out(rank, (uint64_t)j * p.count * es), In(j), a * es);
    }
    if (b) {
        const Work B{BufKind::SCRATCH, 0, b * n, es};
        x.Copy(B.At(rank, (uint64_t)rank * b), In(rank, a * es), b * es, 1);
        Ctx cb{w, x, 1, 0, 0};
        NhrAllGather(cb, all, B);
        for (uint32_t j = 0; j < n; ++j) x.Copy(Out(rank, ((uint64_t)j * p.count + a) * es), B.At(rank, (uint64_t)j * b), b * es, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
}

// AllReduce as ReduceScatter then AllGather over a mesh whose peers sit behind two sets of links (the reference's
// two-die sequence, ins_v2_allreduce_sequence2die_executor.cc:146-343 with the 2-die mesh templates: a package of two
// dies reaches half of its peers through each die's ports).  The peers in my half of the group are served on queue
// 0, those in the other half on queue 1, so both link sets carry data in both phases.  The second queue folds into an
// accumulator of its own in the staging buffer (two queues must not fold into one destination), which joins my slice
// at the end of the phase; the fold order is fixed.  Slices are the flat two-shot slices over all ranks.
HcclResult TwoDieAllReduce(HostWorld& w, HostPrims& x, const Group& all, const Work& wk)
{
    const uint32_t n = all.size();
    if (n == 1) return HCCL_SUCCESS;
    const uint32_t half = (n + 1) / 2;
    auto queueOf = [&](uint32_t j) { return (j < half) == (all.me < half) ? 0u : 1u; };
    uint64_t b, e;
    Slice(wk, n, all.me, &b, &e);
    const uint64_t len = (e - b) * wk.es;
    if (len > w.scratchBytes()) return HCCL_E_MEMORY;
    const uint32_t me = all.world(all.me);
    x.SyncGroup(all.ranks, N_READY);
    bool first = true;
    for (uint32_t k = 1; k < n; ++k) {
        const uint32_t j = (all.me + k) % n;
        if (queueOf(j) == 0) { x.Reduce(wk.At(me, b), wk.At(all.world(j), b), len, 0); continue; }
        if (first) x.Copy(Scratch(me, 0), wk.At(all.world(j), b), len, 1);
        else x.Reduce(Scratch(me, 0), wk.At(all.world(j), b), len, 1);
        first = false;
    }
    if (!first) x.Reduce(wk.At(me, b), Scratch(me, 0), len, 0);
    x.SyncGroup(all.ranks, N_DATA);
    for (uint32_t k = 1; k < n; ++k) {
        const uint32_t j = (all.me + k) % n;
        uint64_t jb, je;
        Slice(wk, n, j, &jb, &je);
        x.Copy(wk.At(me, jb), wk.At(all.world(j), jb), (je - jb) * wk.es, queueOf(j));
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// AllReduce, two-shot over two link sets at once (the reference's AicpuAllReduceSoleMeshConcur,
// ins_v2_all_reduce_two_shot_sole_executor.cc:305-393: ReduceScatter, then AllGather, each with a mesh template
// that spans both link sets): the data is split by the bandwidth of the two sets and each part runs the mesh
// two-shot on its own queue.
void MeshConcurAllReduce(HostWorld& w, HostPrims& x, const Group& all, const Work& wk)
{
    double sa, sb;
    SplitShares(&sa, &sb);
    const uint64_t a = BandwidthSplit(wk.count, sa, sb, std::max<uint64_t>(1, 128 / wk.es));
    const Work A{wk.buf, wk.base, a, wk.es}, B{wk.buf, wk.base + a * wk.es, wk.count - a, wk.es};
    Ctx ca{w, x, 0, 0, 0};
    Ctx cb{w, x, 1, 0, 0};
    if (A.count) MeshReduceScatter(ca, all, A);
    if (B.count) MeshReduceScatter(cb, all, B);
    if (A.count) MeshAllGather(ca, all, A);
    if (B.count) MeshAllGather(cb, all, B);
}

// AlltoAll family: every pair's block is split by the bandwidth of the two link sets; the receiver pulls the first
// parts from its peers in mesh order on queue 0 and the second parts in the opposite order on queue 1 (reference: the
// Concurrent executors of AlltoAll / AlltoAllV, ins_v2_all_to_all_v_concurrent_executor.cc, two mesh templates on two
// link sets).  The senders' displacements are published at the start of their staging buffers.
void ConcurrentAlltoAll(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype), res = DataTypeSize(p.recvType);
    double sa, sb;
    SplitShares(&sa, &sb);
    uint64_t* table = reinterpret_cast<uint64_t*>(w.Resolve(Scratch(rank, 0)));
    for (uint32_t j = 0; j < n; ++j) table[j] = p.sdispls[j] * es;
    x.SyncGroup(all.ranks, N_READY);
    x.Copy(Out(rank, p.rdispls[rank] * res), In(rank, p.sdispls[rank] * es), p.sendCounts[rank] * es);
    for (uint32_t q = 0; q < 2; ++q) {
        for (uint32_t k = 1; k < n; ++k) {
            const uint32_t from = q == 0 ? (rank + k) % n : (rank + n - k) % n;
            const uint64_t sd = reinterpret_cast<const uint64_t*>(w.Resolve(Scratch(from, 0)))[rank];
            const uint64_t a = BandwidthSplit(p.recvCounts[from], sa, sb, 1);
            const uint64_t off = q == 0 ? 0 : a, cnt = q == 0 ? a : p.recvCounts[from] - a;
            if (cnt) x.Copy(Out(rank, (p.rdispls[from] + off) * res), Mem{from, BufKind::INPUT, sd + off * res}, cnt * res, q);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
}

// Scatter: the first part of a rank's block is pulled from the root (reads over the mesh links), the second part is
// pushed by the root into the rank's staging buffer on the second queue (writes over the other link set) and copied
// out locally; a part that does not fit the staging buffer is pulled as well.
void ConcurrentScatter(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t es = DataTypeSize(p.dtype);
    double sa, sb;
    SplitShares(&sa, &sb);
    uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es));
    if ((p.count - a) * es > w.scratchBytes()) a = p.count;
    const uint64_t b = p.count - a, blk = p.count * es;
    x.SyncGroup(all.ranks, N_READY);
    if (a) x.Copy(Out(rank), In(p.root, (uint64_t)rank * blk), a * es, 0);
    if (b) {
        if (rank == p.root)
            for (uint32_t k = 0; k < all.size(); ++k) {
                const uint32_t j = all.world((all.me + k) % all.size());
                x.Copy(j == rank ? Out(rank, a * es) : Scratch(j, 0), In(rank, (uint64_t)j * blk + a * es), b * es, 1);
            }
        x.SyncGroup(all.ranks, N_DATA, 1);
        if (rank != p.root) x.Copy(Out(rank, a * es), Scratch(rank, 0), b * es, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
}

// Broadcast: both parts are scattered from the root (member i takes slice i of a part), then part A is gathered over
// the mesh while part B is gathered by NHR on the second queue.
void ConcurrentBroadcast(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    double sa, sb;
    SplitShares(&sa, &sb);
    const uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es));
    const Work part[2] = {Work{BufKind::OUTPUT, 0, a, es}, Work{BufKind::OUTPUT, a * es, p.count - a, es}};
    x.SyncGroup(all.ranks, N_READY);
    for (uint32_t q = 0; q < 2 && rank != p.root; ++q) {
        uint64_t b, e;
        Slice(part[q], n, rank, &b, &e);
        if (e > b) x.Copy(Out(rank, part[q].base + b * es), Out(p.root, part[q].base + b * es), (e - b) * es, q);
    }
    x.SyncGroup(all.ranks, N_DATA);
    Ctx ca{w, x, 0, 0, 0};
    Ctx cb{w, x, 1, 0, w.scratchBytes()};
    if (part[0].count) AllGatherBy(Fam::MESH, ca, all, part[0]);
    if (part[1].count) AllGatherBy(Fam::NHR, cb, all, part[1]);
}

// Reduce: ReduceScatter of part A over the mesh and of part B by NHR on a copy in the upper half of the staging
// buffer, then the root collects the slices of both parts from their holders.
void ConcurrentReduce(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    double sa, sb;
    SplitShares(&sa, &sb);
    const uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es));
    const uint64_t wOff = w.scratchBytes() / 2;
    x.Copy(Scratch(rank, wOff), In(rank), Bytes(p));
    const Work part[2] = {Work{BufKind::SCRATCH, wOff, a, es}, Work{BufKind::SCRATCH, wOff + a * es, p.count - a, es}};
    Ctx ca{w, x, 0, 0, 0};
    Ctx cb{w, x, 1, 0, w.scratchBytes() / 2};
    if (part[0].count) MeshReduceScatter(ca, all, part[0]);
    if (part[1].count) NhrReduceScatter(cb, all, part[1]);
    x.SyncGroup(all.ranks, N_LEVEL);
    for (uint32_t q = 0; q < 2 && rank == p.root; ++q) {
        for (uint32_t j = 0; j < n; ++j) {
            uint64_t b, e;
            Slice(part[q], n, j, &b, &e);
            if (e > b) x.Copy(Out(rank, part[q].base - wOff + b * es), Scratch(j, part[q].base + b * es), (e - b) * es, q);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
}

// ---------------------------------------------------------------- mesh with a detour (Z-axis detour)
// The reference's mesh templates with a detour (ins_temp_all_gather_mesh_1D_Z_axis_detour.cc and the ReduceScatter /
// Scatter twins) move every pair's slice over TWO channels of the same pair: the direct mesh link and a second channel
// through the other link class, split by bandwidth - p - 1 mesh links against the port count of the second class,
// 8 unless configured (CalcCostCoeff :33-65, CalcDataSplitByBandwidthZAxisDetour template_utils.h:796-805).  Here the
// two parts of a slice run on two queues; HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO="a,b" overrides the shares.
uint64_t DetourDirectPart(uint64_t count, uint32_t ranks, uint32_t es)
{
    const EnvConfig& env = GetEnvConfig();
    double direct = ranks > 1 ? (double)(ranks - 1) : 1.0, detour = 8.0;
    if (env.splitRatio.size() >= 2 && env.splitRatio[0] + env.splitRatio[1] > 0) { direct = env.splitRatio[0]; detour = env.splitRatio[1]; }
    return BandwidthSplit(count, direct, detour, std::max<uint64_t>(1, 128 / es));
}
void DetourAllGather(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    (void)w;
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    const uint64_t a = DetourDirectPart(p.count, n, es), b = p.count - a;
    x.SyncGroup(all.ranks, N_READY);
    for (uint32_t k = 0; k < n; ++k) {
        const uint32_t j = (rank + k) % n;
        if (a) x.Copy(Out(rank, (uint64_t)j * p.count * es), In(j), a * es, 0);
        if (b) x.Copy(Out(rank, ((uint64_t)j * p.count + a) * es), In(j, a * es), b * es, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
}
// ReduceScatter: block `rank` of every peer's input is folded into the output in rank order, the direct part on queue 0
// and the detour part on queue 1 (the two parts are disjoint element ranges).
void DetourReduceScatter(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    (void)w;
    const uint32_t n = all.size(), es = DataTypeSize(p.dtype);
    const uint64_t a = DetourDirectPart(p.count, n, es), b = p.count - a;
    const uint64_t mine = (uint64_t)rank * p.count * es;
    x.SyncGroup(all.ranks, N_READY);
    if (a) x.Copy(Out(rank), In(rank, mine), a * es, 0);
    if (b) x.Copy(Out(rank, a * es), In(rank, mine + a * es), b * es, 1);
    for (uint32_t k = 1; k < n; ++k) {
        const uint32_t j = (rank + k) % n;
        if (a) x.Reduce(Out(rank), In(j, mine), a * es, 0);
        if (b) x.Reduce(Out(rank, a * es), In(j, mine + a * es), b * es, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
}
void DetourScatter(HostWorld& w, HostPrims& x, const Group& all, uint32_t rank, const OpParam& p)
{
    (void)w;
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t a = DetourDirectPart(p.count, all.size(), es), b = p.count - a;
    const uint64_t mine = (uint64_t)rank * p.count * es;
    x.SyncGroup(all.ranks, N_READY);
    if (a) x.Copy(Out(rank), In(p.root, mine), a * es, 0);
    if (b) x.Copy(Out(rank, a * es), In(p.root, mine + a * es), b * es, 1);
    x.SyncGroup(all.ranks, N_DONE);
}

// ---------------------------------------------------------------- two-level Sequence forms of the rooted operators
struct TwoLevel {
    AlgHierarchy h;
    Group g0, g1;                 // my server, my local index across servers
    uint32_t rootLocal = 0;       // local index of the root inside its server
    uint32_t rootServer = 0;      // index of the root's server in level-1 order
    uint32_t relay = 0;           // member of my server that shares the root's local index
    bool flat = false;            // the topology has one level only
};
HcclResult MatchTwoLevel(HostWorld& w, uint32_t rank, uint32_t root, TwoLevel* t)
{
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &t->h));
    t->flat = t->h.levels() < 2;
    if (t->flat) { t->g0 = WholeGroup(w, rank); t->g1.ranks = {rank}; t->g1.me = 0; t->rootLocal = root; t->relay = root; return HCCL_SUCCESS; }
    LevelGroup(t->h, 0, rank, &t->g0);
    LevelGroup(t->h, 1, rank, &t->g1);
    const std::vector<uint32_t>* rs = GroupOf(t->h, 0, root);
    const std::vector<uint32_t>* rl = GroupOf(t->h, 1, root);
    if (!rs || !rl) return HCCL_E_INTERNAL;
    t->rootLocal = IndexIn(*rs, root);
    t->rootServer = IndexIn(*rl, root);
    t->relay = t->g0.world(t->rootLocal);
    return HCCL_SUCCESS;
}

// Broadcast: the root feeds the members of its level-1 group (one per server) by scatter + NHR AllGather, then every
// server spreads the data from that member by scatter + mesh AllGather.
HcclResult SequenceBroadcast(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const Work wk{BufKind::OUTPUT, 0, p.count, es};
    Ctx c{w, x, 0, 0, w.scratchBytes()};
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    if (!t.flat && t.g0.me == t.rootLocal) {
        if (rank != p.root) {
            uint64_t b, e;
            Slice(wk, t.g1.size(), t.g1.me, &b, &e);
            x.Copy(Out(rank, b * es), Out(p.root, b * es), (e - b) * es);
        }
        x.SyncGroup(t.g1.ranks, N_DATA);
        NhrAllGather(c, t.g1, wk);
    }
    x.SyncGroup(t.g0.ranks, N_LEVEL);
    if (rank != t.relay) {
        uint64_t b, e;
        Slice(wk, t.g0.size(), t.g0.me, &b, &e);
        x.Copy(Out(rank, b * es), Out(t.relay, b * es), (e - b) * es);
    }
    x.SyncGroup(t.g0.ranks, N_AUX);
    MeshAllGather(c, t.g0, wk);
    return HCCL_SUCCESS;
}

// Reduce: mesh ReduceScatter inside every server, NHR ReduceScatter across servers on the slice that is left, then the
// root collects the n pieces.
HcclResult SequenceReduce(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t wOff = w.scratchBytes() / 2;
    x.Copy(Scratch(rank, wOff), In(rank), Bytes(p));
    const Work wk{BufKind::SCRATCH, wOff, p.count, es};
    Ctx c{w, x, 0, 0, w.scratchBytes() / 2};
    const Group all = WholeGroup(w, rank);
    MeshReduceScatter(c, t.g0, wk);
    const Work mine = SubWork(wk, t.g0.size(), t.g0.me);
    if (!t.flat) NhrReduceScatter(c, t.g1, mine);
    x.SyncGroup(all.ranks, N_DATA);
    if (rank == p.root) {
        for (uint32_t l = 0; l < t.g0.size(); ++l) {
            const Work sl = SubWork(wk, t.g0.size(), l);
            const std::vector<uint32_t>* col = t.flat ? nullptr : GroupOf(t.h, 1, t.g0.world(l));
            const uint32_t servers = t.flat ? 1 : (uint32_t)col->size();
            for (uint32_t s = 0; s < servers; ++s) {
                const Work piece = SubWork(sl, servers, s);
                const uint32_t holder = t.flat ? t.g0.world(l) : (*col)[s];
                x.Copy(Out(rank, piece.base - wOff), Scratch(holder, piece.base), piece.count * es);
            }
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Scatter: the root hands every server's blocks to the member that shares its local index (level 1), which hands
// them on inside the server (level 0).
HcclResult SequenceScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint64_t blk = Bytes(p);
    if ((uint64_t)t.g0.size() * blk > w.scratchBytes()) {
        HCCL_ERROR("host engine: hierarchical Scatter stages %llu bytes per server, the scratch buffer has %llu", (unsigned long long)(t.g0.size() * blk),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    if (rank == t.relay && rank != p.root)
        for (uint32_t l = 0; l < t.g0.size(); ++l) x.Copy(Scratch(rank, (uint64_t)l * blk), In(p.root, (uint64_t)t.g0.world(l) * blk), blk);
    x.SyncGroup(t.g0.ranks, N_DATA);
    if (t.relay == p.root) x.Copy(Out(rank), In(p.root, (uint64_t)rank * blk), blk);
    else x.Copy(Out(rank), Scratch(t.relay, (uint64_t)t.g0.me * blk), blk);
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Barrier: gather inside the server, dissemination across servers, release inside the server.
HcclResult SequenceBarrier(HostWorld& w, HostPrims& x, uint32_t rank)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, 0, &t));
    x.SyncGroup(t.g0.ranks, N_READY);
    const uint32_t S = t.g1.size();
    for (uint32_t s = 0; s < CeilLog2(S); ++s) {
        const uint32_t d = (1u << s) % S;
        x.Post(t.g1.world((t.g1.me + d) % S), N_LEVEL);
        x.Wait(t.g1.world((t.g1.me + S - d) % S), N_LEVEL);
    }
    x.SyncGroup(t.g0.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- hierarchical AlltoAll / V / VC
// Rank (s, l) = member l of server s.  Stage 1 (inside the server): member l' collects, from every server-mate, the
// blocks bound for the ranks (*, l') and keeps them in scratch ordered by (source member, destination server); blocks for
// itself go straight to its output.  It then publishes where each (source member, destination server) block sits.
// Stage 2 (across servers): rank (s', l') reads that table from every (s, l') and pulls its blocks.  Every block thus
// crosses the inter-server links once, in messages that carry a whole server's contribution.
// Scratch layout per rank: [n send displacements][n send sizes][L x S staging offsets] (bytes, uint64), then the staging.
HcclResult HierAlltoAll(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    const uint32_t n = w.nRanks();
    const Group all = WholeGroup(w, rank);
    Group g0, g1;
    if (h.levels() < 2) { g0 = all; g1.ranks = {rank}; g1.me = 0; }
    else { LevelGroup(h, 0, rank, &g0); LevelGroup(h, 1, rank, &g1); }
    const uint32_t L = g0.size(), S = g1.size();
    const uint32_t es = DataTypeSize(p.dtype), res = DataTypeSize(p.recvType);
    const uint64_t header = ((uint64_t)(2 * n + L * S) * 8 + 127) / 128 * 128;
    auto table = [&](uint32_t r) { return reinterpret_cast<uint64_t*>(w.Resolve(Scratch(r, 0))); };
    uint64_t* mine = table(rank);
    for (uint32_t j = 0; j < n; ++j) { mine[j] = p.sdispls[j] * es; mine[n + j] = p.sendCounts[j] * es; }
    x.SyncGroup(all.ranks, N_READY);
    // stage 1
    uint64_t off = header;
    bool fits = true;
    for (uint32_t l = 0; l < L; ++l) {
        const uint32_t m = g0.world(l);
        const uint64_t* tm = table(m);
        for (uint32_t s = 0; s < S; ++s) {
            const uint32_t d = g1.world(s);
            const uint64_t bytes = tm[n + d];
            mine[2 * n + l * S + s] = off;
            if (d == rank) { x.Copy(Out(rank, p.rdispls[m] * res), In(m, tm[d]), bytes); continue; }
            if (off + bytes > w.scratchBytes()) { fits = false; break; }
            x.Copy(Scratch(rank, off), In(m, tm[d]), bytes);
            off += bytes;
        }
    }
    if (!fits) {
        w.Abort("hierarchical AlltoAll: the blocks relayed by rank " + std::to_string(rank) + " exceed the scratch buffer (raise HCCL_BUFFSIZE)");
        return HCCL_E_MEMORY;
    }
    x.SyncGroup(g1.ranks, N_DATA);
    // stage 2
    for (uint32_t k = 1; k < S; ++k) {
        const uint32_t s = (g1.me + k) % S, relay = g1.world(s);
        const std::vector<uint32_t>* srv = GroupOf(h, 0, relay);
        const uint64_t* tr = table(relay);
        for (uint32_t l = 0; l < L; ++l) {
            const uint32_t src = (*srv)[l];
            x.Copy(Out(rank, p.rdispls[src] * res), Scratch(relay, tr[2 * n + l * S + g1.me]), p.recvCounts[src] * res);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- Pipeline (2-D)
constexpr uint32_t kMaxPipeSteps = 5;

// AllReduce: stage 0 = mesh ReduceScatter inside the server, stage 1 = NHR AllReduce across servers on the slice that
// is left, stage 2 = mesh AllGather inside the server; one queue per stage.
HcclResult PipelineAllReduce(HostWorld& w, HostPrims& x, uint32_t rank, const Work& wk)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    Ctx flat{w, x, 0, 0, w.scratchBytes()};
    if (h.levels() < 2) { AllReduceBy(Fam::MESH, flat, WholeGroup(w, rank), wk); return HCCL_SUCCESS; }
    Group g0, g1;
    LevelGroup(h, 0, rank, &g0);
    LevelGroup(h, 1, rank, &g1);
    const uint32_t steps = PipelineStepCount(wk.count, (uint64_t)g0.size() * g1.size() * std::max<uint64_t>(1, 128 / wk.es), kMaxPipeSteps);
    for (const PipeSlot& s : PipelineSchedule(3, steps)) {
        const Work chunk = SubWork(wk, steps, s.step);
        Ctx c{w, x, s.stage, 0, w.scratchBytes()};
        if (s.stage == 0) MeshReduceScatter(c, g0, chunk);
        else if (s.stage == 1) AllReduceBy(Fam::NHR, c, g1, SubWork(chunk, g0.size(), g0.me));
        else MeshAllGather(c, g0, chunk);
    }
    return HCCL_SUCCESS;
}

// AllReduce on three levels (the reference's 3-D OmniPipe, ins_v2_all_reduce_omnipipe_executor.cc with
// TopoMatchThreeLevel, per-step slices of omnipipe_data_slice_calc.cc): five stages - mesh ReduceScatter inside the
// server, NHR ReduceScatter across the servers of the pod, NHR AllReduce across the pods on the slice that is left,
// NHR AllGather across the servers, mesh AllGather inside the server - each on its own queue, and step i's stage s
// beside step i + 1's stage s - 1.  A topology with fewer levels runs the two-level pipeline.
HcclResult Pipeline3AllReduce(HostWorld& w, HostPrims& x, uint32_t rank, const Work& wk)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::THREE_LEVEL, &h));
    if (h.levels() < 3) return PipelineAllReduce(w, x, rank, wk);
    Group g0, g1, g2;
    LevelGroup(h, 0, rank, &g0);
    LevelGroup(h, 1, rank, &g1);
    LevelGroup(h, 2, rank, &g2);
    const uint64_t ranks = (uint64_t)g0.size() * g1.size() * g2.size();
    const uint32_t steps = PipelineStepCount(wk.count, ranks * std::max<uint64_t>(1, 128 / wk.es), kMaxPipeSteps);
    for (const PipeSlot& s : PipelineSchedule(5, steps)) {
        const Work chunk = SubWork(wk, steps, s.step);
        const Work inServer = SubWork(chunk, g0.size(), g0.me);          // what this rank holds after stage 0
        const Work inPod = SubWork(inServer, g1.size(), g1.me);          // ... and after stage 1
        Ctx c{w, x, s.stage, 0, w.scratchBytes()};
        switch (s.stage) {
            case 0: MeshReduceScatter(c, g0, chunk); break;
            case 1: ReduceScatterBy(Fam::NHR, c, g1, inServer); break;
            case 2: AllReduceBy(Fam::NHR, c, g2, inPod); break;
            case 3: AllGatherBy(Fam::NHR, c, g1, inServer); break;
            default: MeshAllGather(c, g0, chunk); break;
        }
    }
    return HCCL_SUCCESS;
}

// AllGather: every block is cut in steps.  Stage 0 pulls a piece of the server-mates' inputs (mesh), stage 1 pulls the
// same piece of every other server's blocks from the rank with my local index there, once that rank's stage 0 of the
// step is done.  Ranks are numbered server by server.  AllGatherV: block j has its own count and displacement, every
// block is cut in the same number of steps (from the largest block, which all ranks know).
HcclResult PipelineAllGather(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    const Group all = WholeGroup(w, rank);
    Group g0 = all, g1;
    g1.ranks = {rank};
    g1.me = 0;
    if (h.levels() >= 2) { LevelGroup(h, 0, rank, &g0); LevelGroup(h, 1, rank, &g1); }
    const uint32_t es = DataTypeSize(p.dtype);
    const bool v = p.op == HCCL_CMD_ALLGATHER_V;
    auto cnt = [&](uint32_t j) { return v ? p.recvCounts[j] : p.count; };
    auto dsp = [&](uint32_t j) { return v ? p.rdispls[j] : (uint64_t)j * p.count; };
    uint64_t largest = 0;
    for (uint32_t j = 0; j < w.nRanks(); ++j) largest = std::max<uint64_t>(largest, cnt(j));
    const uint32_t steps = PipelineStepCount(largest, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(2, steps)) {
        if (s.stage == 0) {
            for (uint32_t k = 0; k < g0.size(); ++k) {
                const uint32_t j = g0.world((g0.me + k) % g0.size());
                uint64_t b, e;
                SliceOf(cnt(j), steps, s.step, &b, &e);
                if (e > b) x.Copy(Out(rank, (dsp(j) + b) * es), In(j, b * es), (e - b) * es, 0);
            }
        } else {
            x.SyncGroup(g1.ranks, N_DATA, 1);
            for (uint32_t k = 1; k < g1.size(); ++k) {
                const uint32_t peer = g1.world((g1.me + k) % g1.size());
                for (uint32_t j : *GroupOf(h, 0, peer)) {
                    uint64_t b, e;
                    SliceOf(cnt(j), steps, s.step, &b, &e);
                    if (e > b) x.Copy(Out(rank, (dsp(j) + b) * es), Out(peer, (dsp(j) + b) * es), (e - b) * es, 1);
                }
            }
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ReduceScatter, rank (s, l): stage 0 folds, for every server s', the piece of block (s', l) over the members of my
// server into scratch slot s'; stage 1 folds slot s of the ranks (*, l) into my output.
HcclResult PipelineReduceScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    const Group all = WholeGroup(w, rank);
    Group g0 = all, g1;
    g1.ranks = {rank};
    g1.me = 0;
    if (h.levels() >= 2) { LevelGroup(h, 0, rank, &g0); LevelGroup(h, 1, rank, &g1); }
    const uint32_t es = DataTypeSize(p.dtype), S = g1.size();
    const uint64_t blk = p.count * es;
    if ((uint64_t)S * blk > w.scratchBytes()) {
        HCCL_ERROR("host engine: pipelined ReduceScatter stages %llu bytes, the scratch buffer has %llu", (unsigned long long)(S * blk), (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const uint32_t steps = PipelineStepCount(p.count, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(2, steps)) {
        uint64_t b, e;
        SliceOf(p.count, steps, s.step, &b, &e);
        const uint64_t len = (e - b) * es;
        if (s.stage == 0) {
            for (uint32_t t = 0; t < S; ++t) {
                const uint32_t owner = g1.world(t);                 // rank (t, l): the block my partial belongs to
                const Mem slot = Scratch(rank, (uint64_t)t * blk + b * es);
                x.Copy(slot, In(rank, (uint64_t)owner * blk + b * es), len, 0);
                for (uint32_t k = 1; k < g0.size(); ++k) x.Reduce(slot, In(g0.world((g0.me + k) % g0.size()), (uint64_t)owner * blk + b * es), len, 0);
            }
        } else {
            x.SyncGroup(g1.ranks, N_DATA, 1);
            x.Copy(Out(rank, b * es), Scratch(rank, (uint64_t)g1.me * blk + b * es), len, 1);
            for (uint32_t k = 1; k < S; ++k) x.Reduce(Out(rank, b * es), Scratch(g1.world((g1.me + k) % S), (uint64_t)g1.me * blk + b * es), len, 1);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// AllGather on three levels (server, pod, pods): three pipelined stages, one queue each.  Stage 0 pulls a step of the
// server-mates' inputs, stage 1 pulls the same step of the blocks of every other server of the pod from the rank with
// my local index there, stage 2 the blocks of every other pod from the rank at my (server, local) position there -
// each peer hands over exactly what its earlier stages of that step collected.
HcclResult Pipeline3AllGather(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::THREE_LEVEL, &h));
    if (h.levels() < 3) return PipelineAllGather(w, x, rank, p);
    const Group all = WholeGroup(w, rank);
    Group g[3];
    for (uint32_t k = 0; k < 3; ++k) LevelGroup(h, k, rank, &g[k]);
    const uint32_t es = DataTypeSize(p.dtype);
    // the ranks whose blocks `peer` holds when its stages below `level` are done
    std::function<void(uint32_t, uint32_t, std::vector<uint32_t>*)> reach = [&](uint32_t peer, uint32_t level, std::vector<uint32_t>* out) {
        if (level == 0) { out->push_back(peer); return; }
        for (uint32_t m : *GroupOf(h, level - 1, peer)) reach(m, level - 1, out);
    };
    const uint32_t steps = PipelineStepCount(p.count, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(3, steps)) {
        uint64_t b, e;
        SliceOf(p.count, steps, s.step, &b, &e);
        if (s.stage == 0) {
            for (uint32_t k = 0; k < g[0].size(); ++k) {
                const uint32_t j = g[0].world((g[0].me + k) % g[0].size());
                x.Copy(Out(rank, ((uint64_t)j * p.count + b) * es), In(j, b * es), (e - b) * es, 0);
            }
            continue;
        }
        const Group& gs = g[s.stage];
        x.SyncGroup(gs.ranks, s.stage == 1 ? N_DATA : N_AUX, s.stage);
        for (uint32_t k = 1; k < gs.size(); ++k) {
            const uint32_t peer = gs.world((gs.me + k) % gs.size());
            std::vector<uint32_t> blocks;
            reach(peer, s.stage, &blocks);
            for (uint32_t j : blocks) x.Copy(Out(rank, ((uint64_t)j * p.count + b) * es), Out(peer, ((uint64_t)j * p.count + b) * es), (e - b) * es, s.stage);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ReduceScatter on three levels, rank (pod, server, local): stage 0 folds, for every rank q with my local index, a step
// of block q over the members of my server into staging slot (server of q, pod of q); stage 1 folds, for every pod,
// the slot (my server, that pod) of the ranks with my local index in my pod into a second row of slots; stage 2 folds
// my pod's slot of the ranks at my position in the other pods into the output.
HcclResult Pipeline3ReduceScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::THREE_LEVEL, &h));
    if (h.levels() < 3) return PipelineReduceScatter(w, x, rank, p);
    const Group all = WholeGroup(w, rank);
    Group g0, g1, g2;
    LevelGroup(h, 0, rank, &g0);
    LevelGroup(h, 1, rank, &g1);
    LevelGroup(h, 2, rank, &g2);
    const uint32_t es = DataTypeSize(p.dtype), S = g1.size(), P = g2.size();
    const uint64_t blk = p.count * es;
    const uint64_t row1 = (uint64_t)S * P * blk;                    // the second row of slots starts here
    if (row1 + (uint64_t)P * blk > w.scratchBytes()) {
        HCCL_ERROR("host engine: three-level pipelined ReduceScatter stages %llu bytes, the scratch buffer has %llu", (unsigned long long)(row1 + P * blk),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const uint32_t steps = PipelineStepCount(p.count, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(3, steps)) {
        uint64_t b, e;
        SliceOf(p.count, steps, s.step, &b, &e);
        const uint64_t off = b * es, len = (e - b) * es;
        if (s.stage == 0) {
            for (uint32_t i1 = 0; i1 < S; ++i1) {
                const std::vector<uint32_t>* across = GroupOf(h, 2, g1.world(i1));      // the ranks at position (server i1, my local) in every pod
                for (uint32_t i2 = 0; i2 < P; ++i2) {
                    const uint32_t owner = (*across)[i2];
                    const Mem slot = Scratch(rank, ((uint64_t)i1 * P + i2) * blk + off);
                    x.Copy(slot, In(rank, (uint64_t)owner * blk + off), len, 0);
                    for (uint32_t k = 1; k < g0.size(); ++k) x.Reduce(slot, In(g0.world((g0.me + k) % g0.size()), (uint64_t)owner * blk + off), len, 0);
                }
            }
        } else if (s.stage == 1) {
            x.SyncGroup(g1.ranks, N_DATA, 1);
            for (uint32_t i2 = 0; i2 < P; ++i2) {
                const Mem slot = Scratch(rank, row1 + (uint64_t)i2 * blk + off);
                const uint64_t from = ((uint64_t)g1.me * P + i2) * blk + off;
                x.Copy(slot, Scratch(rank, from), len, 1);
                for (uint32_t k = 1; k < S; ++k) x.Reduce(slot, Scratch(g1.world((g1.me + k) % S), from), len, 1);
            }
        } else {
            x.SyncGroup(g2.ranks, N_AUX, 2);
            const uint64_t from = row1 + (uint64_t)g2.me * blk + off;
            x.Copy(Out(rank, off), Scratch(rank, from), len, 2);
            for (uint32_t k = 1; k < P; ++k) x.Reduce(Out(rank, off), Scratch(g2.world((g2.me + k) % P), from), len, 2);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Broadcast: stage 0 moves a step from the root to the member of every server that shares its local index, stage 1
// spreads the step inside every server.
HcclResult PipelineBroadcast(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint32_t steps = PipelineStepCount(p.count, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(2, steps)) {
        uint64_t b, e;
        SliceOf(p.count, steps, s.step, &b, &e);
        if (s.stage == 0) {
            if (rank == t.relay && rank != p.root) x.Copy(Out(rank, b * es), Out(p.root, b * es), (e - b) * es, 0);
        } else {
            x.SyncGroup(t.g0.ranks, N_DATA, 1);
            if (rank != t.relay) x.Copy(Out(rank, b * es), Out(t.relay, b * es), (e - b) * es, 1);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Reduce: the message, copied to the upper half of the staging buffer, is cut in steps; stage 0 = mesh ReduceScatter
// of a step inside the server, stage 1 = NHR ReduceScatter across servers of the slice this rank is left with, and
// when the last step is through the root collects steps x members x servers pieces from their holders.
HcclResult PipelineReduce(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t wOff = w.scratchBytes() / 2;
    x.Copy(Scratch(rank, wOff), In(rank), Bytes(p));
    const Work wk{BufKind::SCRATCH, wOff, p.count, es};
    const Group all = WholeGroup(w, rank);
    const uint32_t servers = t.flat ? 1 : t.g1.size();
    const uint32_t steps = PipelineStepCount(p.count, (uint64_t)t.g0.size() * servers * std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    for (const PipeSlot& s : PipelineSchedule(2, steps)) {
        const Work chunk = SubWork(wk, steps, s.step);
        Ctx c{w, x, s.stage, 0, w.scratchBytes() / 2};
        if (s.stage == 0) MeshReduceScatter(c, t.g0, chunk);
        else if (!t.flat) NhrReduceScatter(c, t.g1, SubWork(chunk, t.g0.size(), t.g0.me));
    }
    x.SyncGroup(all.ranks, N_DATA);
    if (rank == p.root) {
        for (uint32_t step = 0; step < steps; ++step) {
            const Work chunk = SubWork(wk, steps, step);
            for (uint32_t l = 0; l < t.g0.size(); ++l) {
                const Work sl = SubWork(chunk, t.g0.size(), l);
                const std::vector<uint32_t>* col = t.flat ? nullptr : GroupOf(t.h, 1, t.g0.world(l));
                for (uint32_t s = 0; s < servers; ++s) {
                    const Work piece = SubWork(sl, servers, s);
                    const uint32_t holder = t.flat ? t.g0.world(l) : (*col)[s];
                    x.Copy(Out(rank, piece.base - wOff), Scratch(holder, piece.base), piece.count * es);
                }
            }
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Scatter: every block is cut in steps.  Stage 0 moves a step of the blocks of one server from the root to the member
// of that server that shares the root's local index (into its staging buffer, one slot per member), stage 1 hands the
// step on inside the server; the root's own server reads the root's input directly.
HcclResult PipelineScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t blk = Bytes(p);
    if ((uint64_t)t.g0.size() * blk > w.scratchBytes()) {
        HCCL_ERROR("host engine: pipelined Scatter stages %llu bytes per server, the scratch buffer has %llu", (unsigned long long)(t.g0.size() * blk),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const uint32_t steps = PipelineStepCount(p.count, std::max<uint64_t>(1, 128 / es), kMaxPipeSteps);
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    for (const PipeSlot& s : PipelineSchedule(2, steps)) {
        uint64_t b, e;
        SliceOf(p.count, steps, s.step, &b, &e);
        const uint64_t off = b * es, len = (e - b) * es;
        if (s.stage == 0) {
            if (rank == t.relay && rank != p.root)
                for (uint32_t l = 0; l < t.g0.size(); ++l) x.Copy(Scratch(rank, (uint64_t)l * blk + off), In(p.root, (uint64_t)t.g0.world(l) * blk + off), len, 0);
        } else {
            x.SyncGroup(t.g0.ranks, N_DATA, 1);
            if (t.relay == p.root) x.Copy(Out(rank, off), In(p.root, (uint64_t)rank * blk + off), len, 1);
            else x.Copy(Out(rank, off), Scratch(t.relay, (uint64_t)t.g0.me * blk + off), len, 1);
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- Parallel (AllGather, ReduceScatter)
// The reference's Parallel executors cut the data in two parts by the bandwidth of the two levels; part A takes the
// levels bottom-up while part B takes them top-down at the same time, so that both link classes are busy from the
// first step (CalcParallelDataSplitRatio, template_utils.h:809-826; ins_v2_all_gather_parallel_executor.cc and its
// ReduceScatter twin).  Here part A runs on queue 0 with (first, second) = (my server, my column) and part B on queue 1
// with (my column, my server); a column = the ranks that share my local index, one per server.  Both parts of a block
// are element ranges [lo, hi) of it.

// AllGather of the range [lo, hi) of every block: pull it from the members of `first`, wait for the members of
// `second`, pull from each of them what it gathered from ITS `first` group.
void TwoStageAllGather(HostPrims& x, const AlgHierarchy& h, uint32_t firstLevel, const Group& first, const Group& second, uint32_t rank, const OpParam& p,
                       uint64_t lo, uint64_t hi, uint32_t queue, uint32_t notify)
{
    const uint32_t es = DataTypeSize(p.dtype);
    if (hi <= lo) return;
    const uint64_t len = (hi - lo) * es;
    for (uint32_t k = 0; k < first.size(); ++k) {
        const uint32_t j = first.world((first.me + k) % first.size());
        x.Copy(Out(rank, ((uint64_t)j * p.count + lo) * es), In(j, lo * es), len, queue);
    }
    x.SyncGroup(second.ranks, notify, queue);
    for (uint32_t k = 1; k < second.size(); ++k) {
        const uint32_t peer = second.world((second.me + k) % second.size());
        for (uint32_t j : *GroupOf(h, firstLevel, peer)) x.Copy(Out(rank, ((uint64_t)j * p.count + lo) * es), Out(peer, ((uint64_t)j * p.count + lo) * es), len, queue);
    }
}

HcclResult ParallelAllGather(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    if (h.levels() < 2) {
        Group self;
        self.ranks = {rank};
        self.me = 0;
        AlgHierarchy flat;
        flat.infos = {{all.ranks}};
        TwoStageAllGather(x, flat, 0, all, self, rank, p, 0, p.count, 0, N_DATA);
    } else {
        Group g0, g1;
        LevelGroup(h, 0, rank, &g0);
        LevelGroup(h, 1, rank, &g1);
        double sa, sb;
        SplitShares(&sa, &sb);
        const uint64_t a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / DataTypeSize(p.dtype)));
        TwoStageAllGather(x, h, 0, g0, g1, rank, p, 0, a, 0, N_DATA);
        TwoStageAllGather(x, h, 1, g1, g0, rank, p, a, p.count, 1, N_AUX);
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ReduceScatter of the range [lo, hi) of every block: for every member t of `second`, fold the range of ITS block
// over the members of `first` into slot t of my staging region (at scratchOff); wait for the members of `second`; fold
// my slot of theirs into the output.
void TwoStageReduceScatter(HostPrims& x, const Group& first, const Group& second, uint32_t rank, const OpParam& p, uint64_t lo, uint64_t hi,
                           uint64_t scratchOff, uint32_t queue, uint32_t notify)
{
    const uint32_t es = DataTypeSize(p.dtype);
    if (hi <= lo) return;
    const uint64_t len = (hi - lo) * es, blk = p.count * es;
    for (uint32_t t = 0; t < second.size(); ++t) {
        const uint32_t owner = second.world(t);
        const Mem slot = Scratch(rank, scratchOff + (uint64_t)t * len);
        x.Copy(slot, In(rank, (uint64_t)owner * blk + lo * es), len, queue);
        for (uint32_t k = 1; k < first.size(); ++k) x.Reduce(slot, In(first.world((first.me + k) % first.size()), (uint64_t)owner * blk + lo * es), len, queue);
    }
    x.SyncGroup(second.ranks, notify, queue);
    x.Copy(Out(rank, lo * es), Scratch(rank, scratchOff + (uint64_t)second.me * len), len, queue);
    for (uint32_t k = 1; k < second.size(); ++k)
        x.Reduce(Out(rank, lo * es), Scratch(second.world((second.me + k) % second.size()), scratchOff + (uint64_t)second.me * len), len, queue);
}

HcclResult ParallelReduceScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    AlgHierarchy h;
    CHK_RET(MatchTopo(w.Topo(rank), TopoMatchKind::TWO_LEVEL, &h));
    const Group all = WholeGroup(w, rank);
    const uint32_t es = DataTypeSize(p.dtype);
    Group g0 = all, g1;
    g1.ranks = {rank};
    g1.me = 0;
    uint64_t a = p.count;
    if (h.levels() >= 2) {
        LevelGroup(h, 0, rank, &g0);
        LevelGroup(h, 1, rank, &g1);
        double sa, sb;
        SplitShares(&sa, &sb);
        a = BandwidthSplit(p.count, sa, sb, std::max<uint64_t>(1, 128 / es));
    }
    const uint64_t needA = (uint64_t)g1.size() * a * es, needB = (uint64_t)g0.size() * (p.count - a) * es;
    if (needA + needB > w.scratchBytes()) {
        HCCL_ERROR("host engine: parallel ReduceScatter stages %llu bytes, the scratch buffer has %llu", (unsigned long long)(needA + needB),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    x.SyncGroup(all.ranks, N_READY);
    TwoStageReduceScatter(x, g0, g1, rank, p, 0, a, 0, 0, N_DATA);
    if (h.levels() >= 2) TwoStageReduceScatter(x, g1, g0, rank, p, a, p.count, needA, 1, N_AUX);
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Parallel forms of the rooted operators (reference: ins_v2_broadcast_parallel_executor.cc, ins_v2_reduce_parallel_
// executor.cc, ins_v2_scatter_parallel_executor.cc): part A crosses the servers first and spreads inside them second,
// part B the other way round, on the second queue.  "Column" = the ranks that share a local index, one per server;
// the column head is its member in the root's server.
uint64_t ParallelSplit(const TwoLevel& t, uint64_t count, uint32_t es)
{
    if (t.flat) return count;
    double sa, sb;
    SplitShares(&sa, &sb);
    return BandwidthSplit(count, sa, sb, std::max<uint64_t>(1, 128 / es));
}

HcclResult ParallelBroadcast(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t a = ParallelSplit(t, p.count, es), lenA = a * es, lenB = (p.count - a) * es;
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    if (lenA) {
        // root -> the member of every server with the root's local index -> its server
        if (!t.flat && rank == t.relay && rank != p.root) x.Copy(Out(rank), Out(p.root), lenA, 0);
        x.SyncGroup(t.g0.ranks, N_DATA, 0);
        if (rank != t.relay) x.Copy(Out(rank), Out(t.relay), lenA, 0);
    }
    if (lenB) {
        // root -> its own server -> every member's column
        const bool rootServer = t.g1.me == t.rootServer;
        const uint32_t head = t.g1.world(t.rootServer);
        if (rootServer && rank != p.root) x.Copy(Out(rank, lenA), Out(p.root, lenA), lenB, 1);
        x.SyncGroup(t.g1.ranks, N_AUX, 1);
        if (!rootServer) x.Copy(Out(rank, lenA), Out(head, lenA), lenB, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

HcclResult ParallelScatter(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t blk = Bytes(p);
    const uint64_t a = ParallelSplit(t, p.count, es), lenA = a * es, lenB = (p.count - a) * es;
    const uint64_t offB = (uint64_t)t.g0.size() * lenA;                 // part B's staging slots follow part A's
    if (offB + (uint64_t)t.g1.size() * lenB > w.scratchBytes()) {
        HCCL_ERROR("host engine: parallel Scatter stages %llu bytes, the scratch buffer has %llu", (unsigned long long)(offB + t.g1.size() * lenB),
                   (unsigned long long)w.scratchBytes());
        return HCCL_E_MEMORY;
    }
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_READY);
    if (lenA) {
        // the blocks of a server go to its member with the root's local index, which hands them on
        if (rank == t.relay && rank != p.root)
            for (uint32_t l = 0; l < t.g0.size(); ++l) x.Copy(Scratch(rank, (uint64_t)l * lenA), In(p.root, (uint64_t)t.g0.world(l) * blk), lenA, 0);
        x.SyncGroup(t.g0.ranks, N_DATA, 0);
        if (t.relay == p.root) x.Copy(Out(rank), In(p.root, (uint64_t)rank * blk), lenA, 0);
        else x.Copy(Out(rank), Scratch(t.relay, (uint64_t)t.g0.me * lenA), lenA, 0);
    }
    if (lenB) {
        // the blocks of a column go to its head in the root's server, which hands them on
        const bool rootServer = t.g1.me == t.rootServer;
        const uint32_t head = t.g1.world(t.rootServer);
        if (rootServer && rank != p.root)
            for (uint32_t s = 0; s < t.g1.size(); ++s) x.Copy(Scratch(rank, offB + (uint64_t)s * lenB), In(p.root, (uint64_t)t.g1.world(s) * blk + lenA), lenB, 1);
        x.SyncGroup(t.g1.ranks, N_AUX, 1);
        if (head == p.root) x.Copy(Out(rank, lenA), In(p.root, (uint64_t)rank * blk + lenA), lenB, 1);
        else x.Copy(Out(rank, lenA), Scratch(head, offB + (uint64_t)t.g1.me * lenB), lenB, 1);
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// Reduce on a copy in the upper half of the staging buffer: part A = mesh ReduceScatter in the server, NHR
// ReduceScatter along the column; part B = NHR along the column first, mesh in the server second; the root collects
// the pieces of both parts from their holders.  One loop handles at most a quarter of the staging buffer (the two
// parts' templates stage side by side in the lower half).
HcclResult ParallelReduce(HostWorld& w, HostPrims& x, uint32_t rank, const OpParam& p)
{
    TwoLevel t;
    CHK_RET(MatchTwoLevel(w, rank, p.root, &t));
    const uint32_t es = DataTypeSize(p.dtype);
    const uint64_t wOff = w.scratchBytes() / 2, quarter = (w.scratchBytes() / 4) & ~(uint64_t)127;
    if (Bytes(p) > quarter) return HCCL_E_MEMORY;
    x.Copy(Scratch(rank, wOff), In(rank), Bytes(p));
    const uint64_t a = ParallelSplit(t, p.count, es);
    const Work A{BufKind::SCRATCH, wOff, a, es}, B{BufKind::SCRATCH, wOff + a * es, p.count - a, es};
    const uint32_t L = t.g0.size(), S = t.flat ? 1 : t.g1.size();
    Ctx ca{w, x, 0, 0, quarter};
    Ctx cb{w, x, 1, quarter, quarter};
    if (A.count) {
        MeshReduceScatter(ca, t.g0, A);
        if (!t.flat) NhrReduceScatter(ca, t.g1, SubWork(A, L, t.g0.me));
    }
    if (B.count) {
        NhrReduceScatter(cb, t.g1, B);
        MeshReduceScatter(cb, t.g0, SubWork(B, S, t.g1.me));
    }
    const Group all = WholeGroup(w, rank);
    x.SyncGroup(all.ranks, N_DATA);
    if (rank == p.root) {
        for (uint32_t l = 0; l < L; ++l) {
            const std::vector<uint32_t>* col = t.flat ? nullptr : GroupOf(t.h, 1, t.g0.world(l));
            for (uint32_t s = 0; s < S; ++s) {
                const uint32_t holder = t.flat ? t.g0.world(l) : (*col)[s];
                const Work pa = SubWork(SubWork(A, L, l), S, s), pb = SubWork(SubWork(B, S, s), L, l);
                if (pa.count) x.Copy(Out(rank, pa.base - wOff), Scratch(holder, pa.base), pa.count * es, 0);
                if (pb.count) x.Copy(Out(rank, pb.base - wOff), Scratch(holder, pb.base), pb.count * es, 1);
            }
        }
    }
    x.SyncGroup(all.ranks, N_DONE);
    return HCCL_SUCCESS;
}

// ---------------------------------------------------------------- tree executor (AllReduce)
struct TreeRun {
    HostWorld& w;
    HostPrims& x;
    const AlgHierarchy& h;
    uint32_t rank;
};

bool LeafFam(const std::string& leaf, Fam* f)
{
    if (leaf == "mesh") *f = Fam::MESH;
    else if (leaf == "ring") *f = Fam::RING;
    else if (leaf == "nhr" || leaf == "nb") *f = Fam::NHR;
    else if (leaf == "rhd") *f = Fam::RHD;
    else return false;
    return true;
}
void LeafReduceScatter(const std::string& leaf, Ctx& c, const Group& g, const Work& wk)
{
    Fam f = Fam::MESH;
    LeafFam(leaf, &f);
    ReduceScatterBy(f, c, g, wk);
}
void LeafAllGather(const std::string& leaf, Ctx& c, const Group& g, const Work& wk)
{
    if (leaf == "nb") { NbAllGather(c, g, wk); return; }
    Fam f = Fam::MESH;
    LeafFam(leaf, &f);
    AllGatherBy(f, c, g, wk);
}
// The ranks that can differ from me only in the given levels, in rank order (one level: that level's group).
Group FlatGroup(const TreeRun& t, const std::vector<uint32_t>& levels)
{
    std::vector<uint32_t> set = {t.rank};
    for (uint32_t l : levels) {
        std::vector<uint32_t> next;
        for (uint32_t r : set)
            for (uint32_t m : *GroupOf(t.h, l, r)) next.push_back(m);
        std::sort(next.begin(), next.end());
        next.erase(std::unique(next.begin(), next.end()), next.end());
        set.swap(next);
    }
    Group g;
    g.ranks = set;
    g.me = IndexIn(set, t.rank);
    return g;
}
// Scratch bytes a subtree may use per byte of its data: every level of a seq works in a region of its own (a template
// such as the ring writes into its neighbour's staging without asking first, so it must not share a region with the
// level before it), and three levels of at least one rank each need at most three times the data.
constexpr uint64_t kTreeScratchPerByte = 3;

void EvalTree(const TreeRun& t, const AlgoTreeNode& n, std::vector<uint32_t> levels, const Work& wk, uint32_t queue, uint64_t scratchOff)
{
    if (wk.count == 0) return;
    switch (n.kind) {
        case AlgoTreeNode::Kind::LEAF: {
            Ctx c{t.w, t.x, queue, scratchOff, wk.count * wk.es};
            const Group g = FlatGroup(t, levels);
            if (n.leaf == "nb") { NhrReduceScatter(c, g, wk); NbAllGather(c, g, wk); }
            else { Fam f = Fam::MESH; LeafFam(n.leaf, &f); AllReduceBy(f, c, g, wk); }
            break;
        }
        case AlgoTreeNode::Kind::REV:
            std::reverse(levels.begin(), levels.end());
            EvalTree(t, *n.kids[0], levels, wk, queue, scratchOff);
            break;
        case AlgoTreeNode::Kind::PAR: {
            double sa = n.shareA, sb = n.shareB;
            if (sa + sb <= 0) SplitShares(&sa, &sb);
            const uint64_t a = BandwidthSplit(wk.count, sa, sb, std::max<uint64_t>(1, 128 / wk.es));
            const Work A{wk.buf, wk.base, a, wk.es}, B{wk.buf, wk.base + a * wk.es, wk.count - a, wk.es};
            EvalTree(t, *n.kids[0], levels, A, queue, scratchOff);
            EvalTree(t, *n.kids[1], levels, B, queue + AlgoTreeQueues(*n.kids[0]), scratchOff + kTreeScratchPerByte * a * wk.es);
            break;
        }
        case AlgoTreeNode::Kind::SEQ: {
            const size_t lower = n.kids.size() - 1;
            std::vector<Group> groups(lower);
            std::vector<Work> works(lower);
            Work cur = wk;
            std::vector<uint64_t> offs(lower);
            uint64_t off = scratchOff;
            for (size_t i = 0; i < lower; ++i) {
                groups[i] = FlatGroup(t, {levels[i]});
                works[i] = cur;
                offs[i] = off;
                Ctx c{t.w, t.x, queue, off, cur.count * cur.es};
                LeafReduceScatter(n.kids[i]->leaf, c, groups[i], cur);
                off += cur.count * cur.es;
                cur = SubWork(cur, groups[i].size(), groups[i].me);
            }
            EvalTree(t, *n.kids[lower], std::vector<uint32_t>(levels.begin() + (long)lower, levels.end()), cur, queue, off);
            for (size_t i = lower; i-- > 0;) {
                Ctx c{t.w, t.x, queue, offs[i], works[i].count * works[i].es};
                LeafAllGather(n.kids[i]->leaf, c, groups[i], works[i]);
            }
            break;
        }
    }
}

HcclResult TreeAllReduce(HostWorld& w, HostPrims& x, uint32_t rank, const Work& wk)
{
    std::unique_ptr<AlgoTreeNode> tree;
    std::string err;
    if (!ParseAlgoTree(GetEnvConfig().algoTree, &tree, &err)) { HCCL_ERROR("HCCL_ALGO_TREE: %s", err.c_str()); return HCCL_E_PARA; }
    AlgHierarchy h;
    const TopoInfo& topo = w.Topo(rank);
    CHK_RET(MatchTopo(topo, topo.nPods > 1 ? TopoMatchKind::THREE_LEVEL : topo.nServers > 1 ? TopoMatchKind::TWO_LEVEL : TopoMatchKind::ONE_LEVEL, &h));
    if (AlgoTreeMinLevels(*tree) > h.levels()) {
        HCCL_ERROR("HCCL_ALGO_TREE '%s' needs %u topology levels, this communicator has %u", AlgoTreeText(*tree).c_str(), AlgoTreeMinLevels(*tree), h.levels());
        return HCCL_E_PARA;
    }
    std::vector<uint32_t> levels(h.levels());
    std::iota(levels.begin(), levels.end(), 0u);
    const TreeRun t{w, x, h, rank};
    EvalTree(t, *tree, levels, wk, 0, 0);
    return HCCL_SUCCESS;
}

}  // namespace

HcclResult RunHostExecutorExt(HostWorld& w, uint32_t rank, int alg, const OpParam& p)
{
    HostPrims x(&w, rank);
    const uint32_t n = w.nRanks();
    const uint32_t es = DataTypeSize(p.dtype);
    const Group all = WholeGroup(w, rank);
    Ctx c{w, x, 0, 0, w.scratchBytes()};
    HcclResult r = HCCL_SUCCESS;
    switch (alg) {
        case HALG_AR_CONCURRENT_MESH_NHR: case HALG_AR_PIPELINE_MESH_NHR: case HALG_AR_PIPELINE3_MESH_NHR_NHR: case HALG_AR_TREE:
        case HALG_AR_SEQ_2DIE_MESH_MESH: case HALG_AR_SOLE_MESH_CONCUR: {
            x.Copy(Out(rank), In(rank), Bytes(p));
            const Work wk{BufKind::OUTPUT, 0, p.count, es};
            if (alg == HALG_AR_CONCURRENT_MESH_NHR) ConcurrentAllReduce(w, x, all, wk);
            else if (alg == HALG_AR_PIPELINE_MESH_NHR) r = PipelineAllReduce(w, x, rank, wk);
            else if (alg == HALG_AR_PIPELINE3_MESH_NHR_NHR) r = Pipeline3AllReduce(w, x, rank, wk);
            else if (alg == HALG_AR_SEQ_2DIE_MESH_MESH) r = TwoDieAllReduce(w, x, all, wk);
            else if (alg == HALG_AR_SOLE_MESH_CONCUR) MeshConcurAllReduce(w, x, all, wk);
            else r = TreeAllReduce(w, x, rank, wk);
            break;
        }
        case HALG_AG_MESH_DETOUR: DetourAllGather(w, x, all, rank, p); break;
        case HALG_RS_MESH_DETOUR: DetourReduceScatter(w, x, all, rank, p); break;
        case HALG_SCATTER_MESH_DETOUR: DetourScatter(w, x, all, rank, p); break;
        case HALG_RS_CONCURRENT_MESH_NHR: ConcurrentReduceScatter(w, x, all, rank, p); break;
        case HALG_AG_CONCURRENT_MESH_NHR: ConcurrentAllGather(w, x, all, rank, p); break;
        case HALG_BCAST_CONCURRENT_MESH_NHR: ConcurrentBroadcast(w, x, all, rank, p); break;
        case HALG_A2A_CONCURRENT_MESH_MESH: ConcurrentAlltoAll(w, x, all, rank, p); break;
        case HALG_SCATTER_CONCURRENT_MESH_MESH: ConcurrentScatter(w, x, all, rank, p); break;
        case HALG_REDUCE_CONCURRENT_MESH_NHR: ConcurrentReduce(w, x, all, rank, p); break;
        case HALG_AG_PIPELINE_MESH_MESH: r = PipelineAllGather(w, x, rank, p); break;
        case HALG_RS_PIPELINE_MESH_MESH: r = PipelineReduceScatter(w, x, rank, p); break;
        case HALG_BCAST_PIPELINE_MESH_MESH: r = PipelineBroadcast(w, x, rank, p); break;
        case HALG_REDUCE_PIPELINE_MESH_NHR: r = PipelineReduce(w, x, rank, p); break;
        case HALG_AG_PIPELINE3_MESH_MESH_MESH: r = Pipeline3AllGather(w, x, rank, p); break;
        case HALG_RS_PIPELINE3_MESH_MESH_MESH: r = Pipeline3ReduceScatter(w, x, rank, p); break;
        case HALG_AG_PARALLEL_MESH_MESH: r = ParallelAllGather(w, x, rank, p); break;
        case HALG_BCAST_PARALLEL_MESH_MESH: r = ParallelBroadcast(w, x, rank, p); break;
        case HALG_SCATTER_PARALLEL_MESH_MESH: r = ParallelScatter(w, x, rank, p); break;
        case HALG_REDUCE_PARALLEL_MESH_NHR: r = ParallelReduce(w, x, rank, p); break;
        case HALG_RS_PARALLEL_MESH_MESH: r = ParallelReduceScatter(w, x, rank, p); break;
        case HALG_SCATTER_PIPELINE_MESH_MESH: r = PipelineScatter(w, x, rank, p); break;
        case HALG_AG_NB: {
            x.Copy(Out(rank, (uint64_t)rank * p.count * es), In(rank), p.count * es);
            NbAllGather(c, all, Work{BufKind::OUTPUT, 0, p.count * n, es});
            break;
        }
        case HALG_BCAST_NB: {
            const Work wk{BufKind::OUTPUT, 0, p.count, es};
            x.SyncGroup(all.ranks, N_READY);
            if (rank != p.root) {
                uint64_t b, e;
                Slice(wk, n, rank, &b, &e);
                x.Copy(Out(rank, b * es), Out(p.root, b * es), (e - b) * es);
            }
            x.SyncGroup(all.ranks, N_DATA);
            NbAllGather(c, all, wk);
            break;
        }
        case HALG_SCATTER_NB: r = NbScatter(w, x, all, rank, p); break;
        case HALG_A2A_HIER: r = HierAlltoAll(w, x, rank, p); break;
        case HALG_BCAST_SEQ_MESH_NHR: r = SequenceBroadcast(w, x, rank, p); break;
        case HALG_REDUCE_SEQ_MESH_NHR: r = SequenceReduce(w, x, rank, p); break;
        case HALG_SCATTER_SEQ_MESH_MESH: r = SequenceScatter(w, x, rank, p); break;
        case HALG_BARRIER_SEQ_MESH_NHR: r = SequenceBarrier(w, x, rank); break;
        default: return HCCL_E_NOT_SUPPORT;
    }
    if (r != HCCL_SUCCESS) return r;
    if (x.failed() || w.aborted()) return HCCL_E_TIMEOUT;
    return HCCL_SUCCESS;
}

}  // namespace hccl
