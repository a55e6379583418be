#include <algorithm>
#include "step_tables.h"

namespace hccl {

uint32_t CeilLog2(uint32_t p)
{
    uint32_t n = 0;
    if (p <= 1) return 0;
    uint32_t v = p - 1;
    while (v) { ++n; v >>= 1; }
    return n;
}
uint32_t FloorPow2(uint32_t p)
{
    uint32_t v = 1;
    while (v * 2 <= p) v *= 2;
    return v;
}

std::vector<NhrStep> NhrReduceScatterSteps(uint32_t p, uint32_t me)
{
    std::vector<NhrStep> out;
    const uint32_t n = CeilLog2(p);
    for (uint32_t s = 0; s < n; ++s) {
        NhrStep st;
        st.step = s;
        const uint32_t delta = 1u << s;
        st.sendTo = (me + p - delta % p) % p;
        st.recvFrom = (me + delta) % p;
        const uint32_t nSlices = (p - 1 + delta) / (2 * delta);
        const uint32_t stride = (2 * delta) % p;
        uint32_t tx = st.sendTo, rx = me;
        for (uint32_t i = 0; i < nSlices; ++i) {
            st.txSlices.push_back(tx);
            st.rxSlices.push_back(rx);
            tx = (tx + p - stride) % p;
            rx = (rx + p - stride) % p;
        }
        out.push_back(std::move(st));
    }
    return out;
}

std::vector<NhrStep> NhrAllGatherSteps(uint32_t p, uint32_t me)
{
    std::vector<NhrStep> out;
    const uint32_t n = CeilLog2(p);
    for (uint32_t s = 0; s < n; ++s) {
        NhrStep st;
        st.step = s;
        const uint32_t delta = 1u << (n - 1 - s);
        st.sendTo = (me + delta) % p;
        st.recvFrom = (me + p - delta % p) % p;
        const uint32_t nSlices = (p - 1 + delta) / (2 * delta);
        const uint32_t stride = (2 * delta) % p;
        uint32_t tx = me, rx = st.recvFrom;
        for (uint32_t i = 0; i < nSlices; ++i) {
            st.txSlices.push_back(tx);
            st.rxSlices.push_back(rx);
            tx = (tx + p - stride) % p;
            rx = (rx + p - stride) % p;
        }
        out.push_back(std::move(st));
    }
    return out;
}

RhdInfo RhdPart1(uint32_t p, uint32_t rank)
{
    RhdInfo i;
    i.p = p;
    i.P = FloorPow2(p);
    i.r = p - i.P;
    i.steps = CeilLog2(i.P);
    if (rank < i.r) { i.representative = true; i.partner = rank + i.r; i.vrank = rank; }
    else if (rank < 2 * i.r) { i.merged = true; i.partner = rank - i.r; i.vrank = rank - i.r; }
    else i.vrank = rank - i.r;
    return i;
}

uint32_t RhdSigma(uint32_t p, uint32_t a)
{
    const uint32_t r = p - FloorPow2(p);
    if (a < r) return 2 * a;
    if (a < 2 * r) return 2 * (a - r) + 1;
    return a;
}
uint32_t RhdSigmaInv(uint32_t p, uint32_t u)
{
    const uint32_t r = p - FloorPow2(p);
    if (u < 2 * r) return (u % 2 == 0) ? u / 2 : (u - 1) / 2 + r;
    return u;
}
uint32_t RhdVirtualToReal(uint32_t p, uint32_t v)
{
    const uint32_t r = p - FloorPow2(p);
    return v < r ? v : v + r;
}
std::pair<uint32_t, uint32_t> RhdUnitRange(uint32_t p, uint32_t a, uint32_t b)
{
    const uint32_t r = p - FloorPow2(p);
    return {a < r ? 2 * a : a + r, b <= r ? 2 * b : b + r};
}

std::vector<RhdStep> RhdReduceScatterSteps(uint32_t p, uint32_t v)
{
    std::vector<RhdStep> out;
    const uint32_t P = FloorPow2(p), n = CeilLog2(P);
    for (uint32_t k = 0; k < n; ++k) {
        const uint32_t dist = P >> (k + 1);
        RhdStep s;
        s.peerVirtual = v ^ dist;
        const uint32_t myBase = v & ~(dist - 1), peerBase = s.peerVirtual & ~(dist - 1);
        auto send = RhdUnitRange(p, peerBase, peerBase + dist), keep = RhdUnitRange(p, myBase, myBase + dist);
        s.sendUnitBegin = send.first; s.sendUnitEnd = send.second;
        s.keepUnitBegin = keep.first; s.keepUnitEnd = keep.second;
        out.push_back(s);
    }
    return out;
}

std::vector<RhdStep> RhdAllGatherSteps(uint32_t p, uint32_t v)
{
    std::vector<RhdStep> out;
    const uint32_t P = FloorPow2(p), n = CeilLog2(P);
    for (uint32_t k = 0; k < n; ++k) {
        const uint32_t dist = 1u << k;
        RhdStep s;
        s.peerVirtual = v ^ dist;
        const uint32_t held = v & ~(dist - 1), other = held ^ dist;
        auto send = RhdUnitRange(p, held, held + dist), recv = RhdUnitRange(p, other, other + dist);
        s.sendUnitBegin = send.first; s.sendUnitEnd = send.second;
        s.keepUnitBegin = recv.first; s.keepUnitEnd = recv.second;
        out.push_back(s);
    }
    return out;
}

std::vector<RingStep> RingReduceScatterSteps(uint32_t p, uint32_t me)
{
    std::vector<RingStep> out;
    for (uint32_t s = 0; s + 1 < p; ++s) out.push_back({(me + 2 * p - s - 1) % p, (me + 2 * p - s - 2) % p});
    return out;
}
std::vector<RingStep> RingAllGatherSteps(uint32_t p, uint32_t me)
{
    std::vector<RingStep> out;
    for (uint32_t s = 0; s + 1 < p; ++s) out.push_back({(me + p - s) % p, (me + 2 * p - s - 1) % p});
    return out;
}

std::vector<PairwiseStep> PairwiseSteps(uint32_t p, uint32_t me)
{
    std::vector<PairwiseStep> out;
    for (uint32_t k = 1; k < p; ++k) out.push_back({(me + k) % p, (me + p - k) % p});
    return out;
}

std::vector<std::pair<uint32_t, uint32_t>> DeterministicFoldOrder(uint32_t count)
{
    std::vector<std::pair<uint32_t, uint32_t>> out;
    uint32_t cur = count;
    while (cur > 1) {
        uint32_t M = 1;
        while (M * 2 < cur) M *= 2;    // largest power of two strictly below cur
        for (uint32_t s = M; s < cur; ++s) out.push_back({s % M, s});
        cur = M;
    }
    return out;
}

void SliceOf(uint64_t count, uint32_t p, uint32_t i, uint64_t* begin, uint64_t* end)
{
    const uint64_t per = (count + p - 1) / p;
    uint64_t b = per * i, e = per * (i + 1);
    if (b > count) b = count;
    if (e > count) e = count;
    *begin = b;
    *end = e;
}

std::vector<BruckStep> BruckAllGatherSteps(uint32_t p, uint32_t me)
{
    std::vector<BruckStep> out;
    for (uint32_t d = 1; d < p; d <<= 1) {
        BruckStep s;
        s.sendTo = (me + p - d % p) % p;
        s.recvFrom = (me + d) % p;
        s.nBlocks = std::min(d, p - d);
        s.firstSendBlock = me;
        s.firstRecvBlock = (me + d) % p;
        out.push_back(s);
    }
    return out;
}

std::vector<TreeScatterStep> BinomialScatterSteps(uint32_t p, uint32_t v)
{
    std::vector<TreeScatterStep> out;
    if (p <= 1) return out;
    for (uint32_t d = 1u << (CeilLog2(p) - 1);; d >>= 1) {
        TreeScatterStep s;
        if (v % (2 * d) == 0 && v + d < p) {
            s.sends = true;
            s.peer = v + d;
            s.firstBlock = v + d;
            s.nBlocks = std::min(v + 2 * d, p) - (v + d);
        } else if (v % (2 * d) == d) {
            s.receives = true;
            s.peer = v - d;
            s.firstBlock = v;
            s.nBlocks = std::min(v + d, p) - v;
        }
        out.push_back(s);
        if (d == 1) break;
    }
    return out;
}

uint64_t BandwidthSplit(uint64_t count, double bwA, double bwB, uint64_t align)
{
    if (align == 0) align = 1;
    if (bwA <= 0 || count == 0) return 0;
    if (bwB <= 0) return count;
    uint64_t a = (uint64_t)((double)count * (bwA / (bwA + bwB))) / align * align;
    if (a < align) return 0;
    if (count - a < align) return count;
    return a;
}

std::vector<PipeSlot> PipelineSchedule(uint32_t stages, uint32_t steps)
{
    std::vector<PipeSlot> out;
    if (stages == 0 || steps == 0) return out;
    for (uint32_t t = 0; t < steps + stages - 1; ++t)
        for (uint32_t st = stages; st-- > 0;)
            if (t >= st && t - st < steps) out.push_back({t, st, t - st});
    return out;
}

uint32_t PipelineStepCount(uint64_t count, uint64_t minElems, uint32_t maxSteps)
{
    if (minElems == 0) minElems = 1;
    const uint64_t n = count / minElems;
    return (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>(n, maxSteps));
}

}  // namespace hccl
