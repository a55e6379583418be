// Step tables of the algorithm templates (pure arithmetic, engine-agnostic).
//
// Behavioural spec taken from the reference:
//   NHR  - ins_temp_all_reduce_nhr.cc:646-738, template_utils.cc:32-40 and
//          docs/en/user_guide/coll_algo_intro/NHR.md: ceil(log2 p) steps for any p;
//          ReduceScatter step s uses delta = 2^s, sends to (me - delta) mod p,
//          receives from (me + delta) mod p, nSlices = (p - 1 + 2^s) / 2^(s+1),
//          tx slices start at `sendTo`, rx slices at `me`, both stepping by
//          -2^(s+1) mod p; AllGather runs the steps in reverse.
//   RHD  - template_utils.cc:52-308 and coll_algo_intro/RHD.md: for
//          p = 2^k + r the first 2r ranks pair t <-> t + r, the low side
//          represents the pair; virtual rank v = rank (rank < r) or rank - r
//          (rank >= 2r); slot permutation sigma(a) = 2a (a < r), 2(a - r) + 1
//          (r <= a < 2r), a otherwise, so that a pair's two shares are adjacent
//          units; virtual range [a, b) covers units [(a < r ? 2a : a + r),
//          (b <= r ? 2b : b + r)); main step k of ReduceScatter uses
//          dist = P >> (k + 1), peer = v XOR dist, sends the peer's aligned half
//          and keeps its own; AllGather mirrors it with dist = 1 << k.
//   Ring - coll_algo_intro/Ring.md: p - 1 steps, one slice to the right per step.
//   Pairwise - coll_algo_intro/Pairwise.md: step k: send to (i + k) mod p,
//          receive from (i - k) mod p.
//   NB   - Nonuniform Bruck (the reference's scatter_nb.cc / AlgTemplateBase
//          and HCCL_ALGO's "NB"): ceil(log2 p) steps for any p; AllGather step s
//          sends the min(2^s, p - 2^s) blocks held so far, starting at the own
//          block, to (me - 2^s) mod p and receives as many from (me + 2^s) mod p.
//          Scatter runs a binomial tree over root-relative ranks from the widest
//          stride down: the holder of relative blocks [v, v + 2d) hands
//          [v + d, min(v + 2d, p)) to relative rank v + d.
//   Data split of the Parallel / Concurrent executors - CalcParallelDataSplitRatio
//          (template_utils.h:809-826): part A gets bwA / (bwA + bwB) of the data,
//          cut on an alignment boundary.
//   Pipeline schedule - docs/en/user_guide/coll_algo_intro/Pipeline.md and
//          rfcs/0003-executor-template-refactor.md:712-747: the data is cut in
//          at most five steps and stage k of step i runs beside stage k - 1 of
//          step i + 1.
//   Deterministic fold - aiv_all_reduce_mesh_1d_oneshot.h:39-72: with M the
//          largest power of two below the live count, slot[s mod M] += slot[s]
//          for s in [M, count), count = M, repeat.
#pragma once
#include <cstdint>
#include <utility>
#include <vector>

namespace hccl {

uint32_t CeilLog2(uint32_t p);           // bit length of p - 1 (0 for p <= 1)
uint32_t FloorPow2(uint32_t p);          // largest power of two <= p

struct NhrStep {
    uint32_t step;
    uint32_t sendTo, recvFrom;
    std::vector<uint32_t> txSlices, rxSlices;
};
std::vector<NhrStep> NhrReduceScatterSteps(uint32_t p, uint32_t me);
std::vector<NhrStep> NhrAllGatherSteps(uint32_t p, uint32_t me);

struct RhdInfo {
    uint32_t p = 1, P = 1, r = 0;        // p = P + r, P a power of two
    uint32_t steps = 0;                  // log2 P
    bool merged = false;                 // this rank sits on the high side of a pair (idle in the main phase)
    bool representative = false;         // this rank carries a merged partner
    uint32_t partner = 0;                // valid when merged or representative
    uint32_t vrank = 0;                  // valid unless merged
};
RhdInfo RhdPart1(uint32_t p, uint32_t rank);
uint32_t RhdSigma(uint32_t p, uint32_t slot);       // real slice -> unit position
uint32_t RhdSigmaInv(uint32_t p, uint32_t unit);    // unit position -> real slice
uint32_t RhdVirtualToReal(uint32_t p, uint32_t v);  // virtual rank -> real rank of the representative
// Unit range covered by the virtual-rank range [a, b).
std::pair<uint32_t, uint32_t> RhdUnitRange(uint32_t p, uint32_t a, uint32_t b);
struct RhdStep {
    uint32_t peerVirtual;
    uint32_t sendUnitBegin, sendUnitEnd;   // units this rank sends
    uint32_t keepUnitBegin, keepUnitEnd;   // ReduceScatter: units it keeps reducing; AllGather: units it receives
};
std::vector<RhdStep> RhdReduceScatterSteps(uint32_t p, uint32_t vrank);
std::vector<RhdStep> RhdAllGatherSteps(uint32_t p, uint32_t vrank);

struct RingStep { uint32_t sendSlice, recvSlice; };
std::vector<RingStep> RingReduceScatterSteps(uint32_t p, uint32_t me);
std::vector<RingStep> RingAllGatherSteps(uint32_t p, uint32_t me);

struct PairwiseStep { uint32_t sendTo, recvFrom; };
std::vector<PairwiseStep> PairwiseSteps(uint32_t p, uint32_t me);

// (dst, src) pairs: slot[dst] op= slot[src], in the order they must be applied.
std::vector<std::pair<uint32_t, uint32_t>> DeterministicFoldOrder(uint32_t count);

// Nonuniform Bruck AllGather: blocks are named by their owner's rank.
struct BruckStep {
    uint32_t sendTo, recvFrom;
    uint32_t firstSendBlock, firstRecvBlock, nBlocks;    // block ranges [first, first + n) mod p
};
std::vector<BruckStep> BruckAllGatherSteps(uint32_t p, uint32_t me);
// Binomial-tree scatter over relative ranks v = (rank - root) mod p.  Each step names relative ranks and blocks.
struct TreeScatterStep {
    bool sends = false, receives = false;
    uint32_t peer = 0;                                   // relative rank of the partner
    uint32_t firstBlock = 0, nBlocks = 0;                // relative blocks that move
};
std::vector<TreeScatterStep> BinomialScatterSteps(uint32_t p, uint32_t vrank);
// Elements of part A when `count` elements are split in proportion bwA : bwB, rounded down to `align` elements
// (part B takes the rest; a part below `align` elements is folded into the other).
uint64_t BandwidthSplit(uint64_t count, double bwA, double bwB, uint64_t align);
// Pipeline of `stages` stages over `steps` data steps: time slot t runs (stage, step = t - stage) for every stage with
// a valid step, later stages first so that a stage frees its buffer before the previous stage refills it.
struct PipeSlot { uint32_t time, stage, step; };
std::vector<PipeSlot> PipelineSchedule(uint32_t stages, uint32_t steps);
// Number of pipeline steps for a message: at most `maxSteps`, each at least `minElems` elements.
uint32_t PipelineStepCount(uint64_t count, uint64_t minElems, uint32_t maxSteps);

// Slice i of `count` elements over p ranks: sliceCount = ceil(count / p); trailing slices may be empty
// (ins_temp_all_reduce_mesh_1D_two_shot.cc:178-201).
void SliceOf(uint64_t count, uint32_t p, uint32_t i, uint64_t* begin, uint64_t* end);

}  // namespace hccl
