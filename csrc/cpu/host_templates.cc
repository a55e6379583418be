// Algorithm templates of the host engine and the executors that compose them.
//
// A template runs one algorithm on one group of ranks (a sub-communicator) over
// a working buffer W that every rank of the group holds at the same place
// (the rank's OUTPUT buffer or a scratch region), the way the reference's
// InsAlgTemplateBase::KernelRun works on TemplateDataParams
// (alg_v2_template_base.h:19-87, template_utils.h:293-357):
//   ReduceScatter(group, W, n): afterwards member i holds the reduced slice i
//   AllGather(group, W, n):     member i enters with slice i valid, all leave with all slices
//   AllReduce = ReduceScatter + AllGather (mesh two-shot, ring, NHR, RHD) or the
//   one-shot mesh with the deterministic fold.
// Executors: Sole (one template on the whole communicator), Sequence (levels one
// after the other: intra ReduceScatter -> inter AllReduce -> intra AllGather,
// reference ins_v2_all_reduce_sequence_executor_aicpu.cc:598-760, two and
// three levels), Parallel (the data is split in two parts that take the levels
// in opposite order on two queues, reference ins_v2_all_reduce_parallel_executor.cc)
// and OrderPreserved (fixed power-of-two fold tree, bitwise reproducible,
// reference order_preserved_common.h, aiv_all_reduce_mesh_1d_oneshot.h:39-72).
#include <algorithm>
#include <numeric>
#include "../core/log.h"
#include "../ops/op_common.h"
#include "../ops/param_check.h"
#include "host_templates.h"
#include "host_world.h"

namespace hccl {
namespace hosttpl {

void Slice(const Work& wk, uint32_t parts, uint32_t i, uint64_t* b, uint64_t* e)
{
    if (wk.vBegin) { *b = wk.vBegin[i]; *e = wk.vBegin[i] + wk.vCount[i]; return; }
    SliceOf(wk.count, parts, i, b, e);
}

// ---------------------------------------------------------------- mesh
// ReduceScatter over a full mesh: every member reads slice `me` from every other member's W and folds it in.
void MeshReduceScatter(Ctx& c, const Group& g, const Work& wk)
{
    if (g.size() == 1) return;
    c.x.SyncGroup(g.ranks, N_READY, c.q);
    uint64_t b, e;
    Slice(wk, g.size(), g.me, &b, &e);
    for (uint32_t k = 1; k < g.size(); ++k) {
        const uint32_t j = (g.me + k) % g.size();
        c.x.Reduce(wk.At(g.world(g.me), b), wk.At(g.world(j), b), (e - b) * wk.es, c.q);
    }
    c.x.SyncGroup(g.ranks, N_DONE, c.q);
}
void MeshAllGather(Ctx& c, const Group& g, const Work& wk)
{
    if (g.size() == 1) return;
    c.x.SyncGroup(g.ranks, N_READY, c.q);
    for (uint32_t k = 1; k < g.size(); ++k) {
        const uint32_t j = (g.me + k) % g.size();
        uint64_t b, e;
        Slice(wk, g.size(), j, &b, &e);
        c.x.Copy(wk.At(g.world(g.me), b), wk.At(g.world(j), b), (e - b) * wk.es, c.q);
    }
    c.x.SyncGroup(g.ranks, N_DONE, c.q);
}
// One-shot AllReduce: every member writes its whole W into slot[me] of every member's scratch, then folds the slots
// in the fixed power-of-two order (identical on all ranks => bitwise identical results).
void MeshOneShotAllReduce(Ctx& c, const Group& g, const Work& wk)
{
    if (g.size() == 1) return;
    const uint64_t bytes = wk.count * wk.es;
    const uint32_t me = g.world(g.me);
    c.x.SyncGroup(g.ranks, N_READY, c.q);     // previous users of the scratch slots are done
    for (uint32_t k = 0; k < g.size(); ++k) {
        const uint32_t j = (g.me + k) % g.size();
        c.x.Copy(Scratch(g.world(j), c.scratchOff + (uint64_t)g.me * bytes), wk.At(me, 0), bytes, c.q);
    }
    c.x.SyncGroup(g.ranks, N_DATA, c.q);
    for (auto& pr : DeterministicFoldOrder(g.size()))
        c.x.Reduce(Scratch(me, c.scratchOff + (uint64_t)pr.first * bytes), Scratch(me, c.scratchOff + (uint64_t)pr.second * bytes), bytes, c.q);
    c.x.Copy(wk.At(me, 0), Scratch(me, c.scratchOff), bytes, c.q);
    c.x.SyncGroup(g.ranks, N_DONE, c.q);
}

// ---------------------------------------------------------------- ring
void RingReduceScatter(Ctx& c, const Group& g, const Work& wk)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const uint32_t me = g.world(g.me), right = g.world((g.me + 1) % p), left = g.world((g.me + p - 1) % p);
    uint64_t slot = 0;                           // largest slice
    for (uint32_t i = 0; i < p; ++i) {
        uint64_t b0, e0;
        Slice(wk, p, i, &b0, &e0);
        slot = std::max(slot, (e0 - b0) * wk.es);
    }
    uint32_t step = 0;
    for (const RingStep& s : RingReduceScatterSteps(p, g.me)) {
        uint64_t sb, se, rb, re;
        Slice(wk, p, s.sendSlice, &sb, &se);
        Slice(wk, p, s.recvSlice, &rb, &re);
        const uint64_t off = c.scratchOff + (uint64_t)(step & 1u) * slot;
        // the receiver must have consumed what was put into this slot two steps ago
        if (step >= 2) c.x.Wait(right, N_ACK, c.q);
        c.x.Copy(Scratch(right, off), wk.At(me, sb), (se - sb) * wk.es, c.q);
        c.x.Post(right, N_DATA, c.q);
        c.x.Wait(left, N_DATA, c.q);
        c.x.Reduce(wk.At(me, rb), Scratch(me, off), (re - rb) * wk.es, c.q);
        c.x.Post(left, N_ACK, c.q);
        ++step;
    }
    // drain the acknowledgements that were not waited for
    for (uint32_t k = 0; k < std::min<uint32_t>(2, p - 1); ++k) c.x.Wait(right, N_ACK, c.q);
}
void RingAllGather(Ctx& c, const Group& g, const Work& wk)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const uint32_t me = g.world(g.me), right = g.world((g.me + 1) % p), left = g.world((g.me + p - 1) % p);
    c.x.Post(left, N_READY, c.q);     // my W may be written
    c.x.Wait(right, N_READY, c.q);
    for (const RingStep& s : RingAllGatherSteps(p, g.me)) {
        uint64_t sb, se;
        Slice(wk, p, s.sendSlice, &sb, &se);
        c.x.Copy(wk.At(right, sb), wk.At(me, sb), (se - sb) * wk.es, c.q);
        c.x.Post(right, N_DATA, c.q);
        c.x.Wait(left, N_DATA, c.q);
    }
    c.x.Post(right, N_DONE, c.q);
    c.x.Wait(left, N_DONE, c.q);
}

// ---------------------------------------------------------------- NHR
void NhrReduceScatter(Ctx& c, const Group& g, const Work& wk)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const uint32_t me = g.world(g.me);
    for (const NhrStep& s : NhrReduceScatterSteps(p, g.me)) {
        const uint32_t to = g.world(s.sendTo), from = g.world(s.recvFrom);
        c.x.Post(from, N_READY, c.q);          // my scratch is free for this step
        c.x.Wait(to, N_READY, c.q);
        for (uint32_t sl : s.txSlices) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Copy(Scratch(to, c.scratchOff + b * wk.es), wk.At(me, b), (e - b) * wk.es, c.q);
        }
        c.x.Post(to, N_DATA, c.q);
        c.x.Wait(from, N_DATA, c.q);
        for (uint32_t sl : s.rxSlices) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Reduce(wk.At(me, b), Scratch(me, c.scratchOff + b * wk.es), (e - b) * wk.es, c.q);
        }
    }
}
void NhrAllGather(Ctx& c, const Group& g, const Work& wk)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const uint32_t me = g.world(g.me);
    for (const NhrStep& s : NhrAllGatherSteps(p, g.me)) {
        const uint32_t to = g.world(s.sendTo), from = g.world(s.recvFrom);
        c.x.Post(from, N_READY, c.q);
        c.x.Wait(to, N_READY, c.q);
        for (uint32_t sl : s.txSlices) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Copy(wk.At(to, b), wk.At(me, b), (e - b) * wk.es, c.q);
        }
        c.x.Post(to, N_DATA, c.q);
        c.x.Wait(from, N_DATA, c.q);
    }
}

// ---------------------------------------------------------------- RHD
// Unit geometry: units are the p real slices in sigma order.  The data stays in W in REAL slice order; a unit range
// is moved slice by slice, which keeps the algorithm's pairing (who sends which units when) identical to the
// reference while avoiding the mirror copy into a sigma-ordered scratch.
void UnitsForEach(uint32_t p, uint32_t ub, uint32_t ue, const std::function<void(uint32_t)>& fn)
{
    for (uint32_t u = ub; u < ue; ++u) fn(RhdSigmaInv(p, u));
}
void RhdReduceScatter(Ctx& c, const Group& g, const Work& wk, bool skipPost)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const RhdInfo info = RhdPart1(p, g.me);
    const uint32_t me = g.world(g.me);
    auto sendSlices = [&](uint32_t toWorld, uint32_t ub, uint32_t ue) {
        UnitsForEach(p, ub, ue, [&](uint32_t sl) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Copy(Scratch(toWorld, c.scratchOff + b * wk.es), wk.At(me, b), (e - b) * wk.es, c.q);
        });
    };
    auto reduceSlices = [&](uint32_t ub, uint32_t ue) {
        UnitsForEach(p, ub, ue, [&](uint32_t sl) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Reduce(wk.At(me, b), Scratch(me, c.scratchOff + b * wk.es), (e - b) * wk.es, c.q);
        });
    };
    // PRE (FULL segment): the merged rank hands everything to its representative
    if (info.merged) {
        const uint32_t rep = g.world(info.partner);
        c.x.Wait(rep, N_READY, c.q);
        sendSlices(rep, 0, p);
        c.x.Post(rep, N_DATA, c.q);
    } else {
        if (info.representative) {
            const uint32_t m = g.world(info.partner);
            c.x.Post(m, N_READY, c.q);
            c.x.Wait(m, N_DATA, c.q);
            reduceSlices(0, p);
        }
        // MAIN: recursive halving among the P virtual ranks
        for (const RhdStep& s : RhdReduceScatterSteps(p, info.vrank)) {
            const uint32_t peer = g.world(RhdVirtualToReal(p, s.peerVirtual));
            c.x.Post(peer, N_READY, c.q);
            c.x.Wait(peer, N_READY, c.q);
            sendSlices(peer, s.sendUnitBegin, s.sendUnitEnd);
            c.x.Post(peer, N_DATA, c.q);
            c.x.Wait(peer, N_DATA, c.q);
            reduceSlices(s.keepUnitBegin, s.keepUnitEnd);
        }
    }
    // POST (SHARE segment): the representative returns the merged rank's own slice
    if (!skipPost) {
        if (info.representative) {
            const uint32_t m = g.world(info.partner);
            uint64_t b, e;
            Slice(wk, p, info.partner, &b, &e);
            c.x.Copy(wk.At(m, b), wk.At(me, b), (e - b) * wk.es, c.q);
            c.x.Post(m, N_DONE, c.q);
        } else if (info.merged) {
            c.x.Wait(g.world(info.partner), N_DONE, c.q);
        }
    }
}
void RhdAllGather(Ctx& c, const Group& g, const Work& wk, bool skipPre)
{
    const uint32_t p = g.size();
    if (p == 1) return;
    const RhdInfo info = RhdPart1(p, g.me);
    const uint32_t me = g.world(g.me);
    auto pushSlices = [&](uint32_t toWorld, uint32_t ub, uint32_t ue) {
        UnitsForEach(p, ub, ue, [&](uint32_t sl) {
            uint64_t b, e;
            Slice(wk, p, sl, &b, &e);
            c.x.Copy(wk.At(toWorld, b), wk.At(me, b), (e - b) * wk.es, c.q);
        });
    };
    // PRE (SHARE): the merged rank gives its slice to the representative
    if (!skipPre) {
        if (info.merged) {
            const uint32_t rep = g.world(info.partner);
            c.x.Wait(rep, N_READY, c.q);
            uint64_t b, e;
            Slice(wk, p, g.me, &b, &e);
            c.x.Copy(wk.At(rep, b), wk.At(me, b), (e - b) * wk.es, c.q);
            c.x.Post(rep, N_DATA, c.q);
        } else if (info.representative) {
            c.x.Post(g.world(info.partner), N_READY, c.q);
            c.x.Wait(g.world(info.partner), N_DATA, c.q);
        }
    }
    if (!info.merged) {
        for (const RhdStep& s : RhdAllGatherSteps(p, info.vrank)) {
            const uint32_t peer = g.world(RhdVirtualToReal(p, s.peerVirtual));
            c.x.Post(peer, N_READY, c.q);
            c.x.Wait(peer, N_READY, c.q);
            pushSlices(peer, s.sendUnitBegin, s.sendUnitEnd);
            c.x.Post(peer, N_DATA, c.q);
            c.x.Wait(peer, N_DATA, c.q);
        }
        // POST (FULL): everything goes back to the merged rank
        if (info.representative) {
            const uint32_t m = g.world(info.partner);
            c.x.Wait(m, N_AUX, c.q);
            pushSlices(m, 0, p);
            c.x.Post(m, N_DONE, c.q);
        }
    } else {
        c.x.Post(g.world(info.partner), N_AUX, c.q);
        c.x.Wait(g.world(info.partner), N_DONE, c.q);
    }
}

// ---------------------------------------------------------------- composition helpers
void ReduceScatterBy(Fam f, Ctx& c, const Group& g, const Work& wk)
{
    switch (f) {
        case Fam::MESH: MeshReduceScatter(c, g, wk); break;
        case Fam::RING: RingReduceScatter(c, g, wk); break;
        case Fam::NHR: NhrReduceScatter(c, g, wk); break;
        case Fam::RHD: RhdReduceScatter(c, g, wk, false); break;
    }
}
void AllGatherBy(Fam f, Ctx& c, const Group& g, const Work& wk)
{
    switch (f) {
        case Fam::MESH: MeshAllGather(c, g, wk); break;
        case Fam::RING: RingAllGather(c, g, wk); break;
        case Fam::NHR: NhrAllGather(c, g, wk); break;
        case Fam::RHD: RhdAllGather(c, g, wk, false); break;
    }
}
void AllReduceBy(Fam f, Ctx& c, const Group& g, const Work& wk)
{
    if (f == Fam::RHD) {
        // the merged ranks sit out the main phases; the representative bridges ReduceScatter and AllGather locally
        // (rhdSkipPost / skipPrePhase of the reference's sequence executor, :700-741)
        RhdReduceScatter(c, g, wk, true);
        RhdAllGather(c, g, wk, true);
        return;
    }
    ReduceScatterBy(f, c, g, wk);
    AllGatherBy(f, c, g, wk);
}

Group WholeGroup(HostWorld& w, uint32_t rank)
{
    Group g;
    g.ranks.resize(w.nRanks());
    std::iota(g.ranks.begin(), g.ranks.end(), 0u);
    g.me = rank;
    return g;
}
bool LevelGroup(const AlgHierarchy& h, uint32_t level, uint32_t rank, Group* out)
{
    for (auto& grp : h.infos[level]) {
        auto it = std::find(grp.begin(), grp.end(), rank);
        if (it != grp.end()) { out->ranks = grp; out->me = (uint32_t)(it - grp.begin()); return true; }
    }
    return false;
}

// The region of `wk` that slice `idx` of `parts` covers, as a Work of its own.
Work SubWork(const Work& wk, uint32_t parts, uint32_t idx)
{
    uint64_t b, e;
    SliceOf(wk.count, parts, idx, &b, &e);
    return Work{wk.buf, wk.base + b * wk.es, e - b, wk.es};
}

// Sequence AllReduce over the levels of `h` on region wk: ReduceScatter down the levels, AllReduce at the top,
// AllGather back up.
void SequenceAllReduce(Ctx& c, const AlgHierarchy& h, uint32_t rank, const Work& wk, const std::vector<Fam>& fam)
{
    std::vector<Group> groups(h.levels());
    std::vector<Work> works(h.levels());
    Work cur = wk;
    const uint32_t top = h.levels() - 1;
    for (uint32_t l = 0; l < h.levels(); ++l) {
        LevelGroup(h, l, rank, &groups[l]);
        works[l] = cur;
        if (l < top) {
            ReduceScatterBy(fam[l], c, groups[l], cur);
            cur = SubWork(cur, groups[l].size(), groups[l].me);
        }
    }
    AllReduceBy(fam[top], c, groups[top], works[top]);
    for (int l = (int)top - 1; l >= 0; --l) AllGatherBy(fam[(size_t)l], c, groups[(size_t)l], works[(size_t)l]);
}

uint64_t Bytes(const OpParam& p) { return p.count * DataTypeSize(p.dtype); }

}  // namespace hosttpl
using namespace hosttpl;

uint64_t HostScratchMultiple(int alg, uint32_t n)
{
    switch (alg) {
        case HALG_AR_MESH_ONESHOT: case HALG_AR_ORDER_PRESERVED: case HALG_RS_ORDER_PRESERVED: return n;
        case HALG_AR_TREE: return 3;      // one staging region per level of the tree
        case HALG_REDUCE_PARALLEL_MESH_NHR: return 2;      // two parts' templates stage side by side
        default: return 1;
    }
}

HcclResult RunHostAlgorithm(HostWorld& w, uint32_t rank, int alg, const OpParam& p)
{
    HostPrims x(&w, rank);
    Ctx c{w, x, 0, 0, w.scratchBytes()};
    const uint32_t n = w.nRanks();
    const uint32_t es = DataTypeSize(p.dtype);
    const Group all = WholeGroup(w, rank);
    auto hierarchy = [&](TopoMatchKind k, AlgHierarchy* h) { return MatchTopo(w.Topo(rank), k, h); };

    switch (alg) {
        // ------------------------------------------------------------ AllReduce
        case HALG_AR_MESH_ONESHOT: case HALG_AR_MESH_TWOSHOT: case HALG_AR_RING: case HALG_AR_RHD: case HALG_AR_NHR:
        case HALG_AR_ORDER_PRESERVED: {
            x.Copy(Out(rank), In(rank), Bytes(p));
            Work wk{BufKind::OUTPUT, 0, p.count, es};
            if (alg == HALG_AR_MESH_ONESHOT || alg == HALG_AR_ORDER_PRESERVED) MeshOneShotAllReduce(c, all, wk);
            else AllReduceBy(alg == HALG_AR_MESH_TWOSHOT ? Fam::MESH : alg == HALG_AR_RING ? Fam::RING : alg == HALG_AR_RHD ? Fam::RHD : Fam::NHR, c, all, wk);
            break;
        }
        case HALG_AR_SEQ_MESH_RING: case HALG_AR_SEQ_MESH_NHR: case HALG_AR_SEQ_MESH_RHD: case HALG_AR_SEQ3_MESH_NHR_NHR: {
            AlgHierarchy h;
            CHK_RET(hierarchy(alg == HALG_AR_SEQ3_MESH_NHR_NHR ? TopoMatchKind::THREE_LEVEL : TopoMatchKind::TWO_LEVEL, &h));
            x.Copy(Out(rank), In(rank), Bytes(p));
            Work wk{BufKind::OUTPUT, 0, p.count, es};
            std::vector<Fam> fam = {Fam::MESH};
            const Fam upper = alg == HALG_AR_SEQ_MESH_RING ? Fam::RING : alg == HALG_AR_SEQ_MESH_RHD ? Fam::RHD : Fam::NHR;
            while (fam.size() < h.levels()) fam.push_back(upper);
            SequenceAllReduce(c, h, rank, wk, fam);
            break;
        }
        case HALG_AR_SEQ_SQUEEZE2D_MESH_MESH: {
            // a flat group laid out as a grid: mesh ReduceScatter along the rows, mesh AllReduce along the columns on
            // the slice that is left, mesh AllGather along the rows - 2 (sqrt p - 1)-ish partners per rank instead of p - 1
            AlgHierarchy h;
            CHK_RET(hierarchy(TopoMatchKind::SQUEEZE_2D, &h));
            x.Copy(Out(rank), In(rank), Bytes(p));
            Work wk{BufKind::OUTPUT, 0, p.count, es};
            SequenceAllReduce(c, h, rank, wk, std::vector<Fam>(h.levels(), Fam::MESH));
            break;
        }
        case HALG_AR_PARALLEL_MESH_NHR: {
            // two halves take the levels in opposite order, each on its own queue; scratch is split between them
            AlgHierarchy h;
            CHK_RET(hierarchy(TopoMatchKind::TWO_LEVEL, &h));
            x.Copy(Out(rank), In(rank), Bytes(p));
            Work wk{BufKind::OUTPUT, 0, p.count, es};
            Work a = SubWork(wk, 2, 0), b = SubWork(wk, 2, 1);
            Ctx ca{w, x, 0, 0, w.scratchBytes() / 2};
            SequenceAllReduce(ca, h, rank, a, {Fam::MESH, Fam::NHR});
            if (h.levels() == 2) {
                AlgHierarchy rev;
                rev.infos = {h.infos[1], h.infos[0]};
                Ctx cb{w, x, 1, w.scratchBytes() / 2, w.scratchBytes() / 2};
                SequenceAllReduce(cb, rev, rank, b, {Fam::NHR, Fam::MESH});
            } else {
                Ctx cb{w, x, 1, w.scratchBytes() / 2, w.scratchBytes() / 2};
                SequenceAllReduce(cb, h, rank, b, {Fam::MESH});
            }
            break;
        }
        // ------------------------------------------------------------ ReduceScatter (+V through the slice of `me`)
        case HALG_RS_MESH: case HALG_RS_RING: case HALG_RS_RHD: case HALG_RS_NHR: case HALG_RS_ORDER_PRESERVED: case HALG_RS_SEQ_MESH_NHR:
        case HALG_RS_SEQ_MESH_RING: case HALG_RS_SEQ_MESH_RHD: case HALG_RS_SEQ3_MESH_NHR_NHR: {
            // work on a scratch copy of the whole input so that the user's send buffer stays intact; layout of W:
            // rank i's block at i * blockElems (V: at its displacement)
            const bool v = p.op == HCCL_CMD_REDUCE_SCATTER_V;
            if (v && alg != HALG_RS_MESH) {
                // variable blocks through ring / RHD / NHR: the whole input is mirrored into scratch and the templates cut
                // it at the callers' displacements
                uint64_t extent = 0;
                for (uint32_t j = 0; j < n; ++j) extent = std::max(extent, p.sdispls[j] + p.sendCounts[j]);
                const uint64_t wOff = w.scratchBytes() / 2;
                if (extent * es > w.scratchBytes() / 2) { HCCL_ERROR("host engine: ReduceScatterV of %llu bytes needs a larger scratch buffer", (unsigned long long)(extent * es)); return HCCL_E_MEMORY; }
                x.Copy(Scratch(rank, wOff), In(rank), extent * es);
                Work wk{BufKind::SCRATCH, wOff, extent, es};
                wk.vBegin = p.sdispls.data();
                wk.vCount = p.sendCounts.data();
                Ctx cc{w, x, 0, 0, w.scratchBytes() / 2};
                ReduceScatterBy(alg == HALG_RS_RING ? Fam::RING : alg == HALG_RS_RHD ? Fam::RHD : Fam::NHR, cc, all, wk);
                x.Copy(Out(rank), Scratch(rank, wOff + p.sdispls[rank] * es), p.sendCounts[rank] * es);
                x.SyncGroup(all.ranks, N_LEVEL);
                break;
            }
            if (v) {
                // variable blocks over the mesh: each member reduces its own block from every peer's INPUT
                x.SyncGroup(all.ranks, N_READY);
                x.Copy(Out(rank), In(rank, p.sdispls[rank] * es), p.sendCounts[rank] * es);
                for (uint32_t k = 1; k < n; ++k) {
                    const uint32_t j = (rank + k) % n;
                    x.Reduce(Out(rank), In(j, p.sdispls[rank] * es), p.sendCounts[rank] * es);
                }
                x.SyncGroup(all.ranks, N_DONE);
                break;
            }
            const uint64_t total = p.count * n;
            const uint64_t wOff = w.scratchBytes() / 2;     // W in the upper half of scratch, algorithm staging in the lower
            x.Copy(Scratch(rank, wOff), In(rank), total * es);
            Work wk{BufKind::SCRATCH, wOff, total, es};
            Ctx cc{w, x, 0, 0, w.scratchBytes() / 2};
            if (alg == HALG_RS_ORDER_PRESERVED) {
                // every member gathers the p copies of its block and folds them in the fixed order
                x.SyncGroup(all.ranks, N_READY);
                for (uint32_t j = 0; j < n; ++j) x.Copy(Scratch(rank, (uint64_t)j * p.count * es), Scratch(j, wOff + (uint64_t)rank * p.count * es), p.count * es);
                for (auto& pr : DeterministicFoldOrder(n)) x.Reduce(Scratch(rank, (uint64_t)pr.first * p.count * es), Scratch(rank, (uint64_t)pr.second * p.count * es), p.count * es);
                x.Copy(Out(rank), Scratch(rank, 0), p.count * es);
                x.SyncGroup(all.ranks, N_DONE);
                break;
            }
            if (alg == HALG_RS_SEQ_MESH_NHR || alg == HALG_RS_SEQ_MESH_RING || alg == HALG_RS_SEQ_MESH_RHD || alg == HALG_RS_SEQ3_MESH_NHR_NHR) {
                // the top level first on whole pod- or server-sized blocks, then down to level 0 inside the server
                const Fam upper = alg == HALG_RS_SEQ_MESH_RING ? Fam::RING : alg == HALG_RS_SEQ_MESH_RHD ? Fam::RHD : Fam::NHR;
                AlgHierarchy h;
                CHK_RET(hierarchy(alg == HALG_RS_SEQ3_MESH_NHR_NHR ? TopoMatchKind::THREE_LEVEL : TopoMatchKind::TWO_LEVEL, &h));
                if (h.levels() == 3) {
                    Group g0, g1, g2;
                    LevelGroup(h, 0, rank, &g0);
                    LevelGroup(h, 1, rank, &g1);
                    LevelGroup(h, 2, rank, &g2);
                    // ranks are numbered pod by pod and server by server inside a pod
                    ReduceScatterBy(upper, cc, g2, wk);
                    const Work pod = SubWork(wk, g2.size(), g2.me);
                    ReduceScatterBy(upper, cc, g1, pod);
                    MeshReduceScatter(cc, g0, SubWork(pod, g1.size(), g1.me));
                } else if (h.levels() == 2) {
                    Group g0, g1;
                    LevelGroup(h, 0, rank, &g0);
                    LevelGroup(h, 1, rank, &g1);
                    // ranks are numbered server by server: blocks of one server are contiguous
                    ReduceScatterBy(upper, cc, g1, wk);
                    Work mine = SubWork(wk, g1.size(), g1.me);
                    MeshReduceScatter(cc, g0, mine);
                } else {
                    MeshReduceScatter(cc, all, wk);
                }
            } else {
                ReduceScatterBy(alg == HALG_RS_MESH ? Fam::MESH : alg == HALG_RS_RING ? Fam::RING : alg == HALG_RS_RHD ? Fam::RHD : Fam::NHR, cc, all, wk);
            }
            x.Copy(Out(rank), Scratch(rank, wOff + (uint64_t)rank * p.count * es), p.count * es);
            x.SyncGroup(all.ranks, N_LEVEL);     // nobody reuses its scratch while a peer may still touch it
            break;
        }
        // ------------------------------------------------------------ AllGather (+V)
        case HALG_AG_MESH: case HALG_AG_RING: case HALG_AG_RHD: case HALG_AG_NHR: case HALG_AG_SEQ_MESH_NHR:
        case HALG_AG_SEQ_MESH_RING: case HALG_AG_SEQ_MESH_RHD: case HALG_AG_SEQ3_MESH_NHR_NHR: {
            const bool v = p.op == HCCL_CMD_ALLGATHER_V;
            if (v && alg != HALG_AG_MESH) {
                // variable blocks through ring / RHD / NHR, in place in the output at the callers' displacements
                uint64_t extent = 0;
                for (uint32_t j = 0; j < n; ++j) extent = std::max(extent, p.rdispls[j] + p.recvCounts[j]);
                x.Copy(Out(rank, p.rdispls[rank] * es), In(rank), p.recvCounts[rank] * es);
                Work wk{BufKind::OUTPUT, 0, extent, es};
                wk.vBegin = p.rdispls.data();
                wk.vCount = p.recvCounts.data();
                AllGatherBy(alg == HALG_AG_RING ? Fam::RING : alg == HALG_AG_RHD ? Fam::RHD : Fam::NHR, c, all, wk);
                break;
            }
            if (v) {
                x.Copy(Out(rank, p.rdispls[rank] * es), In(rank), p.count * es);
                x.SyncGroup(all.ranks, N_READY);
                for (uint32_t k = 1; k < n; ++k) {
                    const uint32_t j = (rank + k) % n;
                    x.Copy(Out(rank, p.rdispls[j] * es), In(j), p.recvCounts[j] * es);
                }
                x.SyncGroup(all.ranks, N_DONE);
                break;
            }
            x.Copy(Out(rank, (uint64_t)rank * p.count * es), In(rank), p.count * es);
            Work wk{BufKind::OUTPUT, 0, p.count * n, es};
            if (alg == HALG_AG_SEQ_MESH_NHR || alg == HALG_AG_SEQ_MESH_RING || alg == HALG_AG_SEQ_MESH_RHD || alg == HALG_AG_SEQ3_MESH_NHR_NHR) {
                const Fam upper = alg == HALG_AG_SEQ_MESH_RING ? Fam::RING : alg == HALG_AG_SEQ_MESH_RHD ? Fam::RHD : Fam::NHR;
                AlgHierarchy h;
                CHK_RET(hierarchy(alg == HALG_AG_SEQ3_MESH_NHR_NHR ? TopoMatchKind::THREE_LEVEL : TopoMatchKind::TWO_LEVEL, &h));
                if (h.levels() == 3) {
                    // bottom-up: the server's blocks, then the pod's, then everything
                    Group g0, g1, g2;
                    LevelGroup(h, 0, rank, &g0);
                    LevelGroup(h, 1, rank, &g1);
                    LevelGroup(h, 2, rank, &g2);
                    const Work pod = SubWork(wk, g2.size(), g2.me);
                    MeshAllGather(c, g0, SubWork(pod, g1.size(), g1.me));
                    AllGatherBy(upper, c, g1, pod);
                    AllGatherBy(upper, c, g2, wk);
                } else if (h.levels() == 2) {
                    Group g0, g1;
                    LevelGroup(h, 0, rank, &g0);
                    LevelGroup(h, 1, rank, &g1);
                    Work mine = SubWork(wk, g1.size(), g1.me);
                    MeshAllGather(c, g0, mine);
                    AllGatherBy(upper, c, g1, wk);
                } else {
                    MeshAllGather(c, all, wk);
                }
            } else {
                AllGatherBy(alg == HALG_AG_MESH ? Fam::MESH : alg == HALG_AG_RING ? Fam::RING : alg == HALG_AG_RHD ? Fam::RHD : Fam::NHR, c, all, wk);
            }
            break;
        }
        // ------------------------------------------------------------ Broadcast
        case HALG_BCAST_MESH_ONESHOT: {
            x.SyncGroup(all.ranks, N_READY);
            if (rank != p.root) x.Copy(Out(rank), Out(p.root), Bytes(p));
            x.SyncGroup(all.ranks, N_DONE);
            break;
        }
        case HALG_BCAST_MESH_TWOSHOT: case HALG_BCAST_NHR: case HALG_BCAST_RING: case HALG_BCAST_RHD: {
            // scatter from the root (member i takes slice i), then AllGather
            Work wk{BufKind::OUTPUT, 0, p.count, es};
            x.SyncGroup(all.ranks, N_READY);
            if (rank != p.root) {
                uint64_t b, e;
                Slice(wk, n, rank, &b, &e);
                x.Copy(Out(rank, b * es), Out(p.root, b * es), (e - b) * es);
            }
            x.SyncGroup(all.ranks, N_DATA);
            AllGatherBy(alg == HALG_BCAST_NHR ? Fam::NHR : alg == HALG_BCAST_RING ? Fam::RING : alg == HALG_BCAST_RHD ? Fam::RHD : Fam::MESH, c, all, wk);
            break;
        }
        // ------------------------------------------------------------ Reduce
        case HALG_REDUCE_MESH_ONESHOT: {
            x.SyncGroup(all.ranks, N_READY);
            if (rank == p.root) {
                x.Copy(Out(rank), In(rank), Bytes(p));
                for (uint32_t k = 1; k < n; ++k) x.Reduce(Out(rank), In((rank + k) % n), Bytes(p));
            }
            x.SyncGroup(all.ranks, N_DONE);
            break;
        }
        case HALG_REDUCE_MESH_TWOSHOT: case HALG_REDUCE_NHR: case HALG_REDUCE_RING: case HALG_REDUCE_RHD: {
            // ReduceScatter on a scratch copy, then the root collects the slices
            const uint64_t wOff = w.scratchBytes() / 2;
            x.Copy(Scratch(rank, wOff), In(rank), Bytes(p));
            Work wk{BufKind::SCRATCH, wOff, p.count, es};
            Ctx cc{w, x, 0, 0, w.scratchBytes() / 2};
            ReduceScatterBy(alg == HALG_REDUCE_NHR ? Fam::NHR : alg == HALG_REDUCE_RING ? Fam::RING : alg == HALG_REDUCE_RHD ? Fam::RHD : Fam::MESH, cc, all, wk);
            x.SyncGroup(all.ranks, N_LEVEL);
            if (rank == p.root) {
                for (uint32_t j = 0; j < n; ++j) {
                    uint64_t b, e;
                    Slice(wk, n, j, &b, &e);
                    x.Copy(Out(rank, b * es), Scratch(j, wOff + b * es), (e - b) * es);
                }
            }
            x.SyncGroup(all.ranks, N_DONE);
            break;
        }
        // ------------------------------------------------------------ Scatter
        case HALG_SCATTER_MESH: case HALG_SCATTER_NHR: case HALG_SCATTER_RING: {
            x.SyncGroup(all.ranks, N_READY);
            if (alg == HALG_SCATTER_RING && n > 2) {
                // the root feeds the ring; every member forwards the blocks of the members behind it
                // (classic p - 1 step ring scatter, reference scatter_ring.cc:19-153), staged through scratch
                const uint32_t dist = (rank + n - p.root) % n;           // hops from the root
                const uint32_t right = (rank + 1) % n, left = (rank + n - 1) % n;
                const uint64_t blk = p.count * es;
                if (rank == p.root) {
                    x.Copy(Out(rank), In(rank, (uint64_t)rank * blk), blk);
                    for (uint32_t d = n - 1; d >= 1; --d) {                 // farthest block first
                        const uint32_t owner = (p.root + d) % n;
                        x.Copy(Scratch(right, (uint64_t)owner * blk), In(rank, (uint64_t)owner * blk), blk);
                        x.Post(right, N_DATA);
                    }
                } else {
                    for (uint32_t d = n - 1; d >= dist; --d) {
                        const uint32_t owner = (p.root + d) % n;
                        x.Wait(left, N_DATA);
                        if (owner == rank) x.Copy(Out(rank), Scratch(rank, (uint64_t)owner * blk), blk);
                        else { x.Copy(Scratch(right, (uint64_t)owner * blk), Scratch(rank, (uint64_t)owner * blk), blk); x.Post(right, N_DATA); }
                        if (d == dist) break;
                    }
                }
            } else if (rank == p.root) {
                x.Copy(Out(rank), In(rank, (uint64_t)rank * p.count * es), p.count * es);
            } else {
                x.Copy(Out(rank), In(p.root, (uint64_t)rank * p.count * es), p.count * es);
            }
            x.SyncGroup(all.ranks, N_DONE);
            break;
        }
        // ------------------------------------------------------------ AlltoAll family
        case HALG_A2A_MESH: case HALG_A2A_PAIRWISE: {
            const uint32_t res = DataTypeSize(p.recvType);
            // publish my send displacements so that receivers can pull: they sit at the start of my scratch
            uint64_t* table = reinterpret_cast<uint64_t*>(w.Resolve(Scratch(rank, 0)));
            for (uint32_t j = 0; j < n; ++j) table[j] = p.sdispls[j] * es;
            x.SyncGroup(all.ranks, N_READY);
            x.Copy(Out(rank, p.rdispls[rank] * res), In(rank, p.sdispls[rank] * es), p.sendCounts[rank] * es);
            auto pull = [&](uint32_t from) {
                const uint64_t sd = reinterpret_cast<const uint64_t*>(w.Resolve(Scratch(from, 0)))[rank];
                x.Copy(Out(rank, p.rdispls[from] * res), Mem{from, BufKind::INPUT, sd}, p.recvCounts[from] * res);
            };
            if (alg == HALG_A2A_PAIRWISE) {
                // one partner per step: no member is the target of two transfers at once
                for (const PairwiseStep& s : PairwiseSteps(n, rank)) {
                    pull(s.recvFrom);
                    x.Post(s.recvFrom, N_ACK);
                    x.Wait(s.sendTo, N_ACK);
                }
            } else {
                for (uint32_t k = 1; k < n; ++k) pull((rank + k) % n);
            }
            x.SyncGroup(all.ranks, N_DONE);
            break;
        }
        case HALG_A2A_SERIAL: {
            // One peer at a time, for links where a rank may hold only one connection's worth of staging memory
            // (reference: the serial sole executor of AlltoAllV, ins_v2_all_to_all_v_serial_sole_executor.cc:113-171,
            // which also pairs rank ^ step and caps a transfer at half the staging buffer).  Step s pairs a rank with
            // rank ^ s, so both ends of a pair choose each other in the same step and no rank serves two peers at
            // once.  A pair moves max(sent, received) bytes in windows of half the staging buffer: the sender copies
            // window k into half k % 2 of ITS buffer and posts, the receiver copies it out and acknowledges, and the
            // sender waits for the acknowledgement of window k - 2 before it fills that half again - staging window
            // k + 1 overlaps the peer's copy of window k.  Nothing but the staging buffer is read by a peer, so the
            // input may be overwritten as soon as the call returns and no closing rendezvous is needed.
            const uint32_t res = DataTypeSize(p.recvType);
            const uint64_t half = (w.scratchBytes() / 2) & ~(uint64_t)63;
            if (half == 0) return HCCL_E_MEMORY;
            x.Copy(Out(rank, p.rdispls[rank] * res), In(rank, p.sdispls[rank] * es), p.sendCounts[rank] * es);
            uint32_t limit = 1;
            while (limit < n) limit <<= 1;
            for (uint32_t step = 1; step < limit; ++step) {
                const uint32_t peer = rank ^ step;
                if (peer >= n) continue;
                const uint64_t sendB = p.sendCounts[peer] * es, recvB = p.recvCounts[peer] * res;
                const uint64_t most = sendB > recvB ? sendB : recvB;          // the same number on both ends of the pair
                const uint64_t windows = (most + half - 1) / half;
                for (uint64_t k = 0; k < windows; ++k) {
                    const uint64_t off = k * half, slot = (k & 1) * half;
                    const uint64_t sn = sendB > off ? (sendB - off < half ? sendB - off : half) : 0;
                    const uint64_t rn = recvB > off ? (recvB - off < half ? recvB - off : half) : 0;
                    if (k >= 2) x.Wait(peer, N_ACK);
                    if (sn) x.Copy(Scratch(rank, slot), In(rank, p.sdispls[peer] * es + off), sn);
                    x.Post(peer, N_DATA);
                    x.Wait(peer, N_DATA);
                    if (rn) x.Copy(Out(rank, p.rdispls[peer] * res + off), Scratch(peer, slot), rn);
                    x.Post(peer, N_ACK);
                }
                for (uint64_t k = 0; k < (windows < 2 ? windows : 2); ++k) x.Wait(peer, N_ACK);   // both halves free for the next peer
            }
            break;
        }
        // ------------------------------------------------------------ point to point
        case HALG_P2P_DIRECT: {
            // sends publish (buffer, bytes) in a per-destination mailbox in scratch and wait for the receiver to copy
            struct Box { const void* buf; uint64_t bytes; };
            for (const HcclSendRecvItem& it : p.items) {
                if (it.sendRecvType != HCCL_SEND) continue;
                Box* box = reinterpret_cast<Box*>(w.Resolve(Scratch(rank, 4096))) + it.remoteRank;
                box->buf = it.buf;
                box->bytes = it.count * DataTypeSize(it.dataType);
                x.Post(it.remoteRank, N_P2P_DATA);
            }
            for (const HcclSendRecvItem& it : p.items) {
                if (it.sendRecvType != HCCL_RECV) continue;
                x.Wait(it.remoteRank, N_P2P_DATA);
                const Box* box = reinterpret_cast<const Box*>(w.Resolve(Scratch(it.remoteRank, 4096))) + rank;
                const uint64_t bytes = it.count * DataTypeSize(it.dataType);
                if (box->bytes != bytes) { w.Abort("send / recv sizes differ between rank " + std::to_string(it.remoteRank) + " and rank " + std::to_string(rank)); return HCCL_E_PARA; }
                memcpy(it.buf, box->buf, bytes);
                x.Post(it.remoteRank, N_P2P_ACK);
            }
            for (const HcclSendRecvItem& it : p.items)
                if (it.sendRecvType == HCCL_SEND) x.Wait(it.remoteRank, N_P2P_ACK);
            break;
        }
        // ------------------------------------------------------------ Barrier
        case HALG_BARRIER_MESH: x.SyncGroup(all.ranks, N_READY); break;
        case HALG_BARRIER_NHR: case HALG_BARRIER_RHD: {
            // dissemination: ceil(log2 p) rounds, round s talks to +- 2^s
            for (uint32_t s = 0; s < CeilLog2(n); ++s) {
                const uint32_t d = (1u << s) % n;
                x.Post((rank + d) % n, N_READY);
                x.Wait((rank + n - d) % n, N_READY);
            }
            break;
        }
        default: {
            const HcclResult r = RunHostExecutorExt(w, rank, alg, p);
            if (r == HCCL_E_NOT_SUPPORT) HCCL_ERROR("host algorithm %d is not implemented", alg);
            return r;
        }
    }
    if (x.failed() || w.aborted()) return HCCL_E_TIMEOUT;
    return HCCL_SUCCESS;
}

}  // namespace hccl
