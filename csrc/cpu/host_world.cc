#include "host_world.h"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <sstream>
#include <thread>
#include "../core/log.h"
#include "../ops/param_check.h"

namespace hccl {

// ------------------------------------------------------------------ element arithmetic on the host
namespace {

float HalfToFloat(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            exp = 127 - 15 + 1;
            while (!(man & 0x400u)) { man <<= 1; --exp; }
            man &= 0x3FFu;
            bits = sign | (exp << 23) | (man << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
uint16_t FloatToHalf(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int32_t exp = (int32_t)((x >> 23) & 0xFFu) - 127 + 15;
    uint32_t man = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFFu) == 0xFFu) return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
    if (exp >= 31) return (uint16_t)(sign | 0x7C00u);
    if (exp <= 0) {
        if (exp < -10) return (uint16_t)sign;
        man |= 0x800000u;
        const uint32_t shift = (uint32_t)(14 - exp);
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (h & 1u))) ++h;
        return (uint16_t)(sign | h);
    }
    uint32_t h = ((uint32_t)exp << 10) | (man >> 13);
    const uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)(sign | h);
}
float Bf16ToFloat(uint16_t b)
{
    uint32_t x = (uint32_t)b << 16;
    float f;
    memcpy(&f, &x, 4);
    return f;
}
uint16_t FloatToBf16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40u);
    x += 0x7FFFu + ((x >> 16) & 1u);
    return (uint16_t)(x >> 16);
}

template <class T>
T Apply(T a, T b, HcclReduceOp op)
{
    switch (op) {
        case HCCL_REDUCE_SUM: return (T)(a + b);
        case HCCL_REDUCE_PROD: return (T)(a * b);
        case HCCL_REDUCE_MAX: return a > b ? a : b;
        default: return a < b ? a : b;
    }
}
template <class T>
void ReduceTyped(void* dst, const void* src, uint64_t n, HcclReduceOp op)
{
    T* d = (T*)dst;
    const T* s = (const T*)src;
    for (uint64_t i = 0; i < n; ++i) d[i] = Apply<T>(d[i], s[i], op);
}
template <float (*L)(uint16_t), uint16_t (*S)(float)>
void Reduce16(void* dst, const void* src, uint64_t n, HcclReduceOp op)
{
    uint16_t* d = (uint16_t*)dst;
    const uint16_t* s = (const uint16_t*)src;
    for (uint64_t i = 0; i < n; ++i) d[i] = S(Apply<float>(L(d[i]), L(s[i]), op));
}

// false: the host engine has no reduction for this data type (the caller fails the operator instead of returning
// unreduced data)
bool HostReduceBytes(void* dst, const void* src, uint64_t bytes, HcclDataType dt, HcclReduceOp op)
{
    const uint64_t n = bytes / DataTypeSize(dt);
    switch (dt) {
        case HCCL_DATA_TYPE_INT8: ReduceTyped<int8_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT16: ReduceTyped<int16_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT32: ReduceTyped<int32_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_INT64: ReduceTyped<int64_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_UINT64: ReduceTyped<uint64_t>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP32: ReduceTyped<float>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP64: ReduceTyped<double>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_FP16: Reduce16<HalfToFloat, FloatToHalf>(dst, src, n, op); break;
        case HCCL_DATA_TYPE_BFP16: Reduce16<Bf16ToFloat, FloatToBf16>(dst, src, n, op); break;
        default: return false;
    }
    return true;
}

}  // namespace

// ------------------------------------------------------------------ HostWorld
HostWorld::HostWorld(uint32_t nRanks, const TopoMeta& meta, uint64_t scratchBytes, uint64_t timeoutNs)
    : n_(nRanks), scratchBytes_(scratchBytes), timeoutNs_(timeoutNs), posted_((size_t)nRanks * nRanks * kNotifyIdx),
      consumed_((size_t)nRanks * nRanks * kNotifyIdx, 0), dropPosts_(nRanks)
{
    for (auto& d : dropPosts_) d.store(0);
    topo_.resize(n_);
    for (uint32_t r = 0; r < n_; ++r) BuildTopoFromMeta(meta, r, &topo_[r]);
    for (uint32_t r = 0; r < n_; ++r) scratch_.emplace_back(new char[scratchBytes_]);
    in_.assign(n_, nullptr);
    out_.assign(n_, nullptr);
    inBytes_.assign(n_, 0);
    outBytes_.assign(n_, 0);
    descs_.resize(n_);
    for (auto& a : posted_) a.store(0);
}
HostWorld::~HostWorld() {}

void HostWorld::Abort(const std::string& why)
{
    bool expect = false;
    if (aborted_.compare_exchange_strong(expect, true)) {
        std::lock_guard<std::mutex> lk(mu_);
        abortWhy_ = why;
        HCCL_ERROR("host world aborted: %s", why.c_str());
    }
    cv_.notify_all();
}

HcclResult HostWorld::BarrierAll(uint32_t rank)
{
    std::unique_lock<std::mutex> lk(mu_);
    if (aborted_.load()) return HCCL_E_REMOTE;
    const uint64_t gen = generation_;
    if (++arrived_ == n_) {
        arrived_ = 0;
        ++generation_;
        cv_.notify_all();
        return HCCL_SUCCESS;
    }
    const bool done = cv_.wait_for(lk, std::chrono::nanoseconds(timeoutNs_), [&] { return generation_ != gen || aborted_.load(); });
    if (aborted_.load()) return HCCL_E_REMOTE;
    if (!done) {
        // a rank never arrived: nobody else may keep waiting for it
        --arrived_;
        lk.unlock();
        Abort("rank " + std::to_string(rank) + " waited " + std::to_string(timeoutNs_ / 1000000) + " ms for the other ranks to call the operator");
        return HCCL_E_TIMEOUT;
    }
    return HCCL_SUCCESS;
}

HcclResult HostWorld::Recover(uint32_t rank)
{
    std::unique_lock<std::mutex> lk(mu_);
    const uint64_t gen = recoverGen_;
    if (++recoverArrived_ == n_) {
        recoverArrived_ = 0;
        arrived_ = 0;
        aborted_.store(false);
        abortWhy_.clear();
        for (auto& a : posted_) a.store(0);
        std::fill(consumed_.begin(), consumed_.end(), 0);
        ++recoverGen_;
        cv_.notify_all();
        return HCCL_SUCCESS;
    }
    if (!cv_.wait_for(lk, std::chrono::nanoseconds(timeoutNs_), [&] { return recoverGen_ != gen; })) {
        --recoverArrived_;
        HCCL_ERROR("rank %u: the other ranks did not reach the retry point within %llu ms", rank, (unsigned long long)(timeoutNs_ / 1000000));
        return HCCL_E_TIMEOUT;
    }
    return HCCL_SUCCESS;
}

static bool SameCall(const HostOpDesc& a, const HostOpDesc& b)
{
    // Send, Recv and BatchSendRecv are one family: a Send on one rank meets a Recv on another
    auto p2p = [](HcclCMDType op) { return op == HCCL_CMD_SEND || op == HCCL_CMD_RECEIVE || op == HCCL_CMD_BATCH_SEND_RECV; };
    if (p2p(a.op) && p2p(b.op)) return true;
    if (a.op != b.op || a.dtype != b.dtype || a.redOp != b.redOp || a.root != b.root) return false;
    switch (a.op) {
        case HCCL_CMD_ALLTOALLV: case HCCL_CMD_SEND: case HCCL_CMD_RECEIVE: case HCCL_CMD_BATCH_SEND_RECV: return true;   // per-rank counts
        case HCCL_CMD_ALLGATHER_V: return a.recvCounts == b.recvCounts && a.rdispls == b.rdispls;
        case HCCL_CMD_REDUCE_SCATTER_V: return a.sendCounts == b.sendCounts && a.sdispls == b.sdispls;
        default: return a.count == b.count;
    }
}

HcclResult HostWorld::Enter(uint32_t rank, const HostOpDesc& d, const void* in, void* out, uint64_t inBytes, uint64_t outBytes)
{
    if (aborted_.load()) return HCCL_E_REMOTE;
    in_[rank] = in; out_[rank] = out; inBytes_[rank] = inBytes; outBytes_[rank] = outBytes; descs_[rank] = d;
    CHK_RET(BarrierAll(rank));
    // cross-rank parameter consistency (reference inconsistent_check.h): every rank checks, so all fail together
    for (uint32_t r = 0; r < n_; ++r) {
        if (!SameCall(descs_[r], descs_[rank])) {
            HCCL_ERROR("host rank %u and rank %u called different operators or parameters (%s count %llu dtype %s vs %s count %llu dtype %s)", rank, r,
                       CmdName(descs_[rank].op), (unsigned long long)descs_[rank].count, DataTypeName(descs_[rank].dtype), CmdName(descs_[r].op),
                       (unsigned long long)descs_[r].count, DataTypeName(descs_[r].dtype));
            return HCCL_E_PARA;
        }
    }
    if (rank == 0) {
        cur_ = d;
        if (tracing_.load()) {
            std::lock_guard<std::mutex> lk(traceMu_);
            OpRecord rec;
            rec.desc = d;
            rec.inBytes = inBytes_;
            rec.outBytes = outBytes_;
            rec.tasks.resize(n_);
            ops_.push_back(std::move(rec));
        }
    }
    return BarrierAll(rank);
}

HcclResult HostWorld::Leave(uint32_t rank) { return BarrierAll(rank); }

char* HostWorld::Resolve(const Mem& m) const
{
    switch (m.buf) {
        case BufKind::INPUT: return (char*)in_[m.rank] + m.off;
        case BufKind::OUTPUT: return (char*)out_[m.rank] + m.off;
        default: return scratch_[m.rank].get() + m.off;
    }
}
uint64_t HostWorld::BufBytes(uint32_t rank, BufKind k) const
{
    switch (k) {
        case BufKind::INPUT: return inBytes_[rank];
        case BufKind::OUTPUT: return outBytes_[rank];
        default: return scratchBytes_;
    }
}

void HostWorld::Post(uint32_t from, uint32_t to, uint32_t idx)
{
    uint32_t left = dropPosts_[from].load();
    while (left > 0)
        if (dropPosts_[from].compare_exchange_weak(left, left - 1)) return;     // lost on the way
    posted_[((size_t)to * n_ + from) * kNotifyIdx + idx].fetch_add(1, std::memory_order_release);
}
bool HostWorld::Wait(uint32_t me, uint32_t from, uint32_t idx)
{
    const size_t k = ((size_t)me * n_ + from) * kNotifyIdx + idx;
    const uint64_t want = ++consumed_[k];
    const auto t0 = std::chrono::steady_clock::now();
    uint32_t spins = 0;
    while (posted_[k].load(std::memory_order_acquire) < want) {
        if (aborted_.load()) return false;
        if ((++spins & 0xFF) == 0) {
            std::this_thread::yield();
            if ((uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now() - t0).count() > timeoutNs_) {
                Abort("rank " + std::to_string(me) + " gave up waiting for notify " + std::to_string(idx) + " from rank " + std::to_string(from));
                return false;
            }
        }
    }
    return true;
}

void HostWorld::TraceBegin()
{
    std::lock_guard<std::mutex> lk(traceMu_);
    ops_.clear();
    tracing_.store(true);
}
void HostWorld::Append(const Task& t)
{
    // each rank appends to its own list of the current op: no lock needed between ranks
    if (!ops_.empty()) ops_.back().tasks[t.rank].push_back(t);
}

// ------------------------------------------------------------------ HostPrims
void HostPrims::Record(const Task& t)
{
    if (w_->tracing()) w_->Append(t);
}

void HostPrims::Copy(Mem dst, Mem src, uint64_t bytes, uint32_t queue)
{
    if (bytes == 0 || failed_) return;
    Task t{};
    t.kind = (dst.rank == me_ && src.rank == me_) ? TaskKind::LOCAL_COPY : (dst.rank == me_ ? TaskKind::READ : TaskKind::WRITE);
    t.rank = me_; t.queue = queue; t.dst = dst; t.src = src; t.bytes = bytes;
    if (dst.rank != me_ && src.rank != me_) { w_->Abort("a rank may only move data from or to itself"); failed_ = true; return; }
    if (dst.off + bytes > w_->BufBytes(dst.rank, dst.buf) || src.off + bytes > w_->BufBytes(src.rank, src.buf)) {
        w_->Abort("copy outside a buffer (rank " + std::to_string(me_) + ")");
        failed_ = true;
        return;
    }
    Record(t);
    memmove(w_->Resolve(dst), w_->Resolve(src), bytes);
}

void HostPrims::Reduce(Mem dst, Mem src, uint64_t bytes, uint32_t queue)
{
    if (bytes == 0 || failed_) return;
    Task t{};
    t.kind = (dst.rank == me_ && src.rank == me_) ? TaskKind::LOCAL_REDUCE : (dst.rank == me_ ? TaskKind::READ_REDUCE : TaskKind::WRITE_REDUCE);
    t.rank = me_; t.queue = queue; t.dst = dst; t.src = src; t.bytes = bytes;
    if (dst.rank != me_ && src.rank != me_) { w_->Abort("a rank may only reduce from or into itself"); failed_ = true; return; }
    if (dst.off + bytes > w_->BufBytes(dst.rank, dst.buf) || src.off + bytes > w_->BufBytes(src.rank, src.buf)) {
        w_->Abort("reduce outside a buffer (rank " + std::to_string(me_) + ")");
        failed_ = true;
        return;
    }
    Record(t);
    const HostOpDesc& d = w_->CurrentOp();
    if (!HostReduceBytes(w_->Resolve(dst), w_->Resolve(src), bytes, d.dtype, d.redOp)) {
        failed_ = true;
        w_->Abort(std::string("the host engine cannot reduce data type ") + DataTypeName(d.dtype));
    }
}

void HostPrims::Post(uint32_t peer, uint32_t idx, uint32_t queue)
{
    if (failed_) return;
    Task t{};
    t.kind = TaskKind::POST; t.rank = me_; t.queue = queue; t.peer = peer; t.notifyIdx = idx;
    Record(t);
    w_->Post(me_, peer, idx);
}
void HostPrims::Wait(uint32_t peer, uint32_t idx, uint32_t queue)
{
    if (failed_) return;
    Task t{};
    t.kind = TaskKind::WAIT; t.rank = me_; t.queue = queue; t.peer = peer; t.notifyIdx = idx;
    Record(t);
    if (!w_->Wait(me_, peer, idx)) failed_ = true;
}
void HostPrims::SyncGroup(const std::vector<uint32_t>& group, uint32_t idx, uint32_t queue)
{
    for (uint32_t r : group) if (r != me_) Post(r, idx, queue);
    for (uint32_t r : group) if (r != me_) Wait(r, idx, queue);
}

std::string VerifyReport::Text() const
{
    std::ostringstream os;
    os << (ok ? "OK" : "FAILED") << ": " << tasks << " tasks (" << dataTasks << " data), " << edges << " ordering edges";
    for (auto& e : errors) os << "\n  " << e;
    return os.str();
}

}  // namespace hccl
