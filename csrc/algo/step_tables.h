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

// Slice i of `count` elements over p ranks: sliceCount = ceil(count / p); trailing slices may be empty
// (ins_temp_all_reduce_mesh_1D_two_shot.cc:178-201).
void SliceOf(uint64_t count, uint32_t p, uint32_t i, uint64_t* begin, uint64_t* end);

}  // namespace hccl
