// Kernel bodies of the collective operators (P2P engine and NVLS engine).
//
// What each body replaces in HCCL: the Mesh1D template family that runs on the
// vector cores and on the CCU - one-shot and two-shot AllReduce
// (aiv_all_reduce_mesh_1d_oneshot.h, aiv_all_reduce_mesh_1d_twoshot.h,
// ccu_kernel_all_reduce_mesh1d_one_shot.cc), mesh ReduceScatter / AllGather /
// Broadcast / Reduce / Scatter / AlltoAll(V) (aiv_reduce_scatter_mesh_1d.h,
// aiv_all_gather_mesh_1d.h, aiv_broadcast_mesh_1d.h, aiv_reduce_mesh_1d.h,
// aiv_scatter_mesh_1d.h, aiv_all_to_all_v_mesh_1D.h).  On one NVSwitch box every
// peer is one hop away at full bandwidth, so the mesh family is the right
// topology class; the design here is pull-based: a rank reads its peers'
// inputs (a registered symmetric buffer, or the copy the peer staged in its
// slab) straight into registers, reduces in rank order 0..p-1 (bitwise
// reproducible on every rank and run) and writes local memory.  Only sources
// have to be peer-visible, destinations never.
//
// Block rows are independent: block b of every rank works on sub-range b of
// every slice and synchronises only with block b of the peers, so no grid-wide
// sync exists and the same code runs as one cooperative launch over all ranks
// when ranks are emulated on one GPU.
#pragma once
#include "dev_comm.cuh"
#include "reduce_ops.cuh"

namespace hccl {

// U vectors per source in flight: the unrolled body of BlockReduceRange for p <= PMAX sources and an aligned destination.
template <class T, int U, int PMAX>
__device__ __forceinline__ void ReduceVecLoop(const char* const* srcs, int p, char* dst, char* const* extra, int nExtra,
                                              size_t head, size_t nv, int op, size_t& i)
{
    const size_t nt = blockDim.x;
    for (; i + (U - 1) * nt < nv; i += U * nt) {
        uint4 raw[U][PMAX];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int q = 0; q < PMAX; ++q)
                if (q < p) raw[u][q] = LdVec(srcs[q] + head + ((i + u * nt) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) {
            AccVec<T> acc;
            Unpack<T>(raw[u][0], acc);
#pragma unroll
            for (int q = 1; q < PMAX; ++q)
                if (q < p) Accumulate<T>(raw[u][q], acc, op);
            const uint4 r = Pack<T>(acc);
            StVec(dst + head + ((i + u * nt) << 4), r);
            for (int x = 0; x < nExtra; ++x) StVec(extra[x] + head + ((i + u * nt) << 4), r);
        }
    }
}

// ---------------------------------------------------------------------------
// Reduce `nBytes` from p equally-aligned sources into dst (and optionally the
// same bytes into nExtra more destinations).  One block, all threads.
template <class T>
__device__ __forceinline__ void BlockReduceRange(const char* const* srcs, int p, char* dst, char* const* extra,
                                                 int nExtra, size_t nBytes, int op)
{
    using Tr = ElemTraits<T>;
    const int tid = threadIdx.x, nt = blockDim.x;
    if (nBytes == 0) return;
    const size_t mis = (uintptr_t)srcs[0] & 15u;
    size_t head = mis ? (16 - mis) : 0;
    if (head > nBytes) head = nBytes;
    // scalar head
    for (size_t e = tid; e < head / sizeof(T); e += nt) {
        typename Tr::Acc acc = Tr::Load(reinterpret_cast<const T*>(srcs[0])[e]);
        for (int q = 1; q < p; ++q) acc = ApplyOp(acc, Tr::Load(reinterpret_cast<const T*>(srcs[q])[e]), op);
        const T r = Tr::Store(acc);
        reinterpret_cast<T*>(dst)[e] = r;
        for (int x = 0; x < nExtra; ++x) reinterpret_cast<T*>(extra[x])[e] = r;
    }
    const size_t nv = (nBytes - head) >> 4;
    const bool dstAligned = (((uintptr_t)(dst + head)) & 15u) == 0;
    size_t i = tid;
    // bulk: eight (small groups) or sixteen loads in flight per thread; the remainder goes one vector at a time
    if (dstAligned) {
        if (p <= 2) ReduceVecLoop<T, 4, 2>(srcs, p, dst, extra, nExtra, head, nv, op, i);
        else if (p <= 4) ReduceVecLoop<T, 2, 4>(srcs, p, dst, extra, nExtra, head, nv, op, i);
        else ReduceVecLoop<T, 2, kMaxDevRanks>(srcs, p, dst, extra, nExtra, head, nv, op, i);
    }
    for (; i < nv; i += nt) {
        uint4 raw[kMaxDevRanks];
#pragma unroll
        for (int q = 0; q < kMaxDevRanks; ++q)
            if (q < p) raw[q] = LdVec(srcs[q] + head + (i << 4));
        AccVec<T> acc;
        Unpack<T>(raw[0], acc);
#pragma unroll
        for (int q = 1; q < kMaxDevRanks; ++q)
            if (q < p) Accumulate<T>(raw[q], acc, op);
        const uint4 r = Pack<T>(acc);
        if (dstAligned) {
            StVec(dst + head + (i << 4), r);
        } else {
            const T* e = reinterpret_cast<const T*>(&r);
            T* d = reinterpret_cast<T*>(dst + head + (i << 4));
#pragma unroll
            for (int k = 0; k < Tr::N; ++k) d[k] = e[k];
        }
        for (int x = 0; x < nExtra; ++x) StVec(extra[x] + head + (i << 4), r);  // extras share src alignment
    }
    // scalar tail
    const size_t done = head + (nv << 4);
    for (size_t e = done / sizeof(T) + tid; e < nBytes / sizeof(T); e += nt) {
        typename Tr::Acc acc = Tr::Load(reinterpret_cast<const T*>(srcs[0])[e]);
        for (int q = 1; q < p; ++q) acc = ApplyOp(acc, Tr::Load(reinterpret_cast<const T*>(srcs[q])[e]), op);
        const T r = Tr::Store(acc);
        reinterpret_cast<T*>(dst)[e] = r;
        for (int x = 0; x < nExtra; ++x) reinterpret_cast<T*>(extra[x])[e] = r;
    }
}

// Slice s of `bytes` split over p ranks in units of 16 bytes (the last slice takes
// the remainder, trailing slices may be empty: reference slicing rule
// ins_temp_all_reduce_mesh_1D_two_shot.cc:178-201), then sub-range b of nb blocks.
__device__ __forceinline__ void SliceSub(size_t bytes, int p, int s, int nb, int b, size_t* off, size_t* len)
{
    size_t sb, se;
    Share(bytes, p, s, 16, &sb, &se);
    size_t bb, be;
    Share(se - sb, nb, b, 16, &bb, &be);
    *off = sb + bb;
    *len = be - bb;
}

// ---------------------------------------------------------------------------
// Barrier
struct BarrierBody {
    using Args = CollArgs;
    static constexpr int kThreads = 64;
    __device__ static void Run(const DevComm& c, const Args&, int b, int)
    {
        OpHead(c, b);
        const uint64_t e = LoadEpoch(c, b);
        RankBarrier(c, b, 0, e + 1, K_BARRIER);
        StoreEpoch(c, b, e + 1);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// AllReduce, two-shot.  bytes = whole message.  Sync points: 3.
template <class T>
struct ArTwoShotBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            for (int s = 0; s < p; ++s) {
                size_t off, len;
                SliceSub(a.bytes, p, s, nb, b, &off, &len);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, len);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_AR_TWOSHOT);
        size_t off, len;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        const char* srcs[kMaxDevRanks];
        for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + off;
        if (a.mode & MODE_PUSH) {
            char* extra[kMaxDevRanks];
            int n = 0;
            for (int q = 1; q < p; ++q) extra[n++] = a.dst[(me + q) % p] + off;
            BlockReduceRange<T>(srcs, p, a.dst[me] + off, extra, n, len, a.op);
            RankBarrier(c, b, 0, e + 2, K_AR_TWOSHOT);
            StoreEpoch(c, b, e + 2);
            OpTail(c, b);
            return;
        }
        const bool direct = !(a.mode & MODE_STAGE_OUT);
        {
            char* extra[1] = {a.out + off};
            BlockReduceRange<T>(srcs, p, a.xch[me] + off, extra, direct ? 1 : 0, len, a.op);
        }
        RankBarrier(c, b, 0, e + 2, K_AR_TWOSHOT);
        {
            CopySeg segs[kMaxDevRanks];
            int n = 0;
            for (int k = direct ? 1 : 0; k < p; ++k) {
                const int q = (me + k) % p;
                size_t qo, ql;
                SliceSub(a.bytes, p, q, nb, b, &qo, &ql);
                segs[n++] = CopySeg{a.out + qo, a.xch[q] + qo, ql};
            }
            BlockCopyMulti(segs, n);
        }
        RankBarrier(c, b, 0, e + 3, K_AR_TWOSHOT);
        StoreEpoch(c, b, e + 3);
        OpTail(c, b);
    }
};

// AllReduce, one-shot pull: every rank reads the whole message from every peer.
// Sync points: 2.
template <class T>
struct ArOneShotBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        size_t off, end;
        Share(a.bytes, nb, b, 16, &off, &end);
        if (a.mode & MODE_STAGE_IN) BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, end - off);
        RankBarrier(c, b, 0, e + 1, K_AR_ONESHOT);
        const char* srcs[kMaxDevRanks];
        for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + off;
        BlockReduceRange<T>(srcs, p, a.out + off, nullptr, 0, end - off, a.op);
        RankBarrier(c, b, 0, e + 2, K_AR_ONESHOT);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// LL (flag-in-data) protocol.  A 16-byte line carries 8 payload bytes:
// {data0, flag, data1, flag}; a line is valid when both flags equal the op's
// flag value.  Writers store lines into the READER's LL slot [parity][writer].
__device__ __forceinline__ char* LLSlot(const DevComm& c, int owner, int parity, int writer)
{
    return c.slab[owner] + kSlabLLOff + ((size_t)(parity * kMaxDevRanks + writer)) * kLLSlotBytes;
}
#ifdef HCCL_HOST_SHIM
// a line is two 8-byte halves {data, flag}; each half is written and read as one atomic unit, as the 16-byte
// volatile vector access is on the GPU
inline void LLStore(char* line, uint32_t d0, uint32_t d1, uint32_t flag)
{
    __atomic_store_n(reinterpret_cast<uint64_t*>(line), (uint64_t)d0 | ((uint64_t)flag << 32), __ATOMIC_RELAXED);
    __atomic_store_n(reinterpret_cast<uint64_t*>(line) + 1, (uint64_t)d1 | ((uint64_t)flag << 32), __ATOMIC_RELAXED);
}
inline uint4 LLPeek(const char* line)
{
    const uint64_t lo = __atomic_load_n(reinterpret_cast<const uint64_t*>(line), __ATOMIC_RELAXED);
    const uint64_t hi = __atomic_load_n(reinterpret_cast<const uint64_t*>(line) + 1, __ATOMIC_RELAXED);
    return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, (uint32_t)(hi >> 32));
}
#else
__device__ __forceinline__ void LLStore(char* line, uint32_t d0, uint32_t d1, uint32_t flag)
{
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(line), "r"(d0), "r"(flag), "r"(d1), "r"(flag)
                 : "memory");
}
// One read of a line without waiting: {data0, flag, data1, flag}.
__device__ __forceinline__ uint4 LLPeek(const char* line)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(line) : "memory");
    return v;
}
#endif
__device__ __forceinline__ bool LLLoad(const DevComm& c, const char* line, uint32_t flag, uint32_t* d0, uint32_t* d1,
                                       uint32_t kernelId, int block, int peer)
{
    uint32_t a, f0, bb, f1;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    for (;;) {
        const uint4 v = LLPeek(line);
        a = v.x; f0 = v.y; bb = v.z; f1 = v.w;
        if (f0 == flag && f1 == flag) break;
        HCCL_SPIN_PAUSE();
        if ((++spins & 0x3FFu) == 0u) {
            if (LdVolatileU32(c.abortWord) != 0u) return false;
            const uint64_t now = GlobalTimerNs();
            if (t0 == 0) t0 = now;
            else if (now - t0 > c.timeoutNs) {
                ReportWaitFailure(c, kernelId, block, 0, peer, flag, f0, DEV_ERR_TIMEOUT);
                return false;
            }
        }
    }
    *d0 = a;
    *d1 = bb;
    return true;
}
__device__ __forceinline__ uint32_t LLFlag(uint64_t epoch) { return (uint32_t)(epoch % 0xFFFFFFFFull) + 1u; }

// Loads up to 8 payload bytes [off, off+8) of `base` (clamped at `bytes`) as two words.
__device__ __forceinline__ void LoadPayload8(const char* base, size_t off, size_t bytes, bool aligned8, uint32_t* d0,
                                             uint32_t* d1)
{
    if (aligned8 && off + 8 <= bytes) {
        const uint2 v = *reinterpret_cast<const uint2*>(base + off);
        *d0 = v.x;
        *d1 = v.y;
        return;
    }
    uint32_t w[2] = {0u, 0u};
    unsigned char* wb = reinterpret_cast<unsigned char*>(w);
    for (int k = 0; k < 8; ++k)
        if (off + k < bytes) wb[k] = (unsigned char)base[off + k];
    *d0 = w[0];
    *d1 = w[1];
}
__device__ __forceinline__ void StorePayload8(char* base, size_t off, size_t bytes, bool aligned8, uint32_t d0,
                                              uint32_t d1)
{
    if (aligned8 && off + 8 <= bytes) {
        *reinterpret_cast<uint2*>(base + off) = make_uint2(d0, d1);
        return;
    }
    uint32_t w[2] = {d0, d1};
    const unsigned char* wb = reinterpret_cast<const unsigned char*>(w);
    for (int k = 0; k < 8; ++k)
        if (off + k < bytes) base[off + k] = (char)wb[k];
}

// AllReduce LL one-shot: bytes <= kLLMaxPayload.
template <class T>
struct ArLLBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        using Tr = ElemTraits<T>;
        constexpr int EPL = 8 / (int)sizeof(T);  // elements per line
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t ep = LoadLLEpoch(c);
        const uint32_t flag = LLFlag(ep);
        const int parity = (int)(ep & 1u);
        const size_t nLines = (a.bytes + 7) >> 3;
        size_t lb, le;
        Share(nLines, nb, b, 1, &lb, &le);
        LLCreditWait(c, ep, K_AR_LL, b);
        const bool inAl = (((uintptr_t)a.in) & 7u) == 0, outAl = (((uintptr_t)a.out) & 7u) == 0;
        for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
            uint32_t d0, d1;
            LoadPayload8(a.in, i << 3, a.bytes, inAl, &d0, &d1);
            for (int k = 0; k < p; ++k) {
                const int q = (me + k) % p;
                LLStore(LLSlot(c, q, parity, me) + (i << 4), d0, d1, flag);
            }
        }
        for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
            // first try: the lines of all peers are requested together, so one memory latency covers them; only a
            // line that has not arrived yet is polled
            uint4 raw[kMaxDevRanks];
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q)
                if (q < p) raw[q] = LLPeek(LLSlot(c, me, parity, q) + (i << 4));
            typename Tr::Acc acc[EPL];
            bool ok = true;
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q) {
                if (q < p) {
                    uint32_t w[2] = {raw[q].x, raw[q].z};
                    if (raw[q].y != flag || raw[q].w != flag)
                        ok = ok && LLLoad(c, LLSlot(c, me, parity, q) + (i << 4), flag, &w[0], &w[1], K_AR_LL, b, q);
                    const T* el = reinterpret_cast<const T*>(w);
#pragma unroll
                    for (int k = 0; k < EPL; ++k) acc[k] = q == 0 ? Tr::Load(el[k]) : ApplyOp(acc[k], Tr::Load(el[k]), a.op);
                }
            }
            uint32_t r[2];
            T* rl = reinterpret_cast<T*>(r);
#pragma unroll
            for (int k = 0; k < EPL; ++k) rl[k] = Tr::Store(acc[k]);
            if (ok) StorePayload8(a.out, i << 3, a.bytes, outAl, r[0], r[1]);
        }
        FinishLLEpoch(c, ep, nb);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// NVLS primitives (multimem.*): the switch reduces / replicates.
template <class T>
struct Multimem;  // only the specialisations below exist
#ifdef HCCL_HOST_SHIM
// the switch's reduction / replication as loops over the ranks' copies (plain accesses: races stay visible)
template <class T>
struct MultimemHost {
    static uint4 LdReduceAdd(const void* mc)
    {
        size_t off = 0;
        const hostshim::McWindow* w = hostshim::McFind(mc, &off);
        AccVec<T> acc;
        for (size_t r = 0; r < w->targets.size(); ++r) {
            const uint4 raw = *reinterpret_cast<const uint4*>(w->targets[r] + off);
            if (r == 0) Unpack<T>(raw, acc);
            else Accumulate<T>(raw, acc, RED_SUM);
        }
        return Pack<T>(acc);
    }
};
template <> struct Multimem<float> : MultimemHost<float> {};
template <> struct Multimem<__nv_bfloat16> : MultimemHost<__nv_bfloat16> {};
template <> struct Multimem<__half> : MultimemHost<__half> {};
inline void MultimemSt(void* mc, const uint4& v)
{
    size_t off = 0;
    const hostshim::McWindow* w = hostshim::McFind(mc, &off);
    for (char* t : w->targets) *reinterpret_cast<uint4*>(t + off) = v;
}
#else
template <>
struct Multimem<float> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void* mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
        return v;
    }
};
template <>
struct Multimem<__nv_bfloat16> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void* mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
        return v;
    }
};
template <>
struct Multimem<__half> {
    __device__ static __forceinline__ uint4 LdReduceAdd(const void* mc)
    {
        uint4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "l"(mc)
                     : "memory");
        return v;
    }
};
__device__ __forceinline__ void MultimemSt(void* mc, const uint4& v)
{
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
#endif

// AllReduce NVLS (sum of fp32 / bf16 / fp16): each rank ld_reduces its slice
// through the switch and multimem-stores the result to every rank.  Requires
// 16-byte aligned, multicast-bound src (user symmetric buffer or the slab) and
// dst (same).  bytes % 16 tail is reduced with plain peer loads.  Sync points: 2,
// plus the copy-out when results were staged.
template <class T>
struct ArNvlsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            for (int s = 0; s < p; ++s) {
                size_t off, len;
                SliceSub(a.bytes, p, s, nb, b, &off, &len);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, len);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_AR_NVLS);
        size_t off, len;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        const size_t nv = len >> 4;
        {
            // eight switch reductions in flight per thread
            size_t i = threadIdx.x;
            const size_t st = blockDim.x;
            for (; i + 7 * st < nv; i += 8 * st) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = Multimem<T>::LdReduceAdd(a.srcMc + off + ((i + u * st) << 4));
#pragma unroll
                for (int u = 0; u < 8; ++u) MultimemSt(a.dstMc + off + ((i + u * st) << 4), v[u]);
            }
            for (; i < nv; i += st) {
                const uint4 v = Multimem<T>::LdReduceAdd(a.srcMc + off + (i << 4));
                MultimemSt(a.dstMc + off + (i << 4), v);
            }
        }
        if (len & 15u) {  // only the very last sub-range of the last slice can have one
            const size_t to = off + (nv << 4);
            const char* srcs[kMaxDevRanks];
            for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + to;
            char* extra[kMaxDevRanks];
            int n = 0;
            for (int q = 1; q < p; ++q) extra[n++] = a.dst[(me + q) % p] + to;
            BlockReduceRange<T>(srcs, p, a.dst[me] + to, extra, n, len & 15u, RED_SUM);
        }
        RankBarrier(c, b, 0, e + 2, K_AR_NVLS);
        if (a.mode & MODE_STAGE_OUT) {
            for (int s = 0; s < p; ++s) {
                size_t so, sl;
                SliceSub(a.bytes, p, s, nb, b, &so, &sl);
                BlockCopyBytes(a.out + so, a.dst[me] + so, sl);
            }
        }
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// ReduceScatter (and V): this rank reduces bytes [dsp[me], dsp[me]+cnt[me]) of
// every rank's peer-visible input into `out`.  Sync points: 2.  With
// MODE_STAGE_IN block q of the local input (at in + dsp2[q]) is first copied
// to src[me] + dsp[q].
template <class T>
struct RsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            // stage exactly the byte ranges peers will read: range q, sub-range b
            for (int q = 0; q < p; ++q) {
                size_t sb, se;
                Share(a.cnt[q], nb, b, 16, &sb, &se);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + a.dsp[q] + sb, a.in + a.dsp2[q] + sb, se - sb);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_RS);
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        const char* srcs[kMaxDevRanks];
        for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + a.dsp[me] + sb;
        BlockReduceRange<T>(srcs, p, a.out + sb, nullptr, 0, se - sb, a.op);
        RankBarrier(c, b, 0, e + 2, K_RS);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ReduceScatter NVLS (sum; fp32/bf16/fp16): ld_reduce of this rank's range.
template <class T>
struct RsNvlsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            for (int q = 0; q < p; ++q) {
                size_t sb, se;
                Share(a.cnt[q], nb, b, 16, &sb, &se);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + a.dsp[q] + sb, a.in + a.dsp2[q] + sb, se - sb);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_RS_NVLS);
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        const size_t base = a.dsp[me] + sb;          // host guarantees 16-byte alignment of dsp
        const size_t nv = (se - sb) >> 4;
        const bool outAl = (((uintptr_t)(a.out + sb)) & 15u) == 0;
        size_t i0 = threadIdx.x;
        if (outAl) {
            const size_t st = blockDim.x;
            for (; i0 + 7 * st < nv; i0 += 8 * st) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = Multimem<T>::LdReduceAdd(a.srcMc + base + ((i0 + u * st) << 4));
#pragma unroll
                for (int u = 0; u < 8; ++u) StVec(a.out + sb + ((i0 + u * st) << 4), v[u]);
            }
        }
        for (size_t i = i0; i < nv; i += blockDim.x) {
            const uint4 v = Multimem<T>::LdReduceAdd(a.srcMc + base + (i << 4));
            if (outAl) {
                StVec(a.out + sb + (i << 4), v);
            } else {
                const T* el = reinterpret_cast<const T*>(&v);
                T* d = reinterpret_cast<T*>(a.out + sb + (i << 4));
#pragma unroll
                for (int k = 0; k < ElemTraits<T>::N; ++k) d[k] = el[k];
            }
        }
        if ((se - sb) & 15u) {
            const char* srcs[kMaxDevRanks];
            for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + base + (nv << 4);
            BlockReduceRange<T>(srcs, p, a.out + sb + (nv << 4), nullptr, 0, (se - sb) & 15u, RED_SUM);
        }
        RankBarrier(c, b, 0, e + 2, K_RS_NVLS);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// AllGather (and V): out[dsp[q] .. +cnt[q]) = rank q's input (cnt[q] bytes).
// Sync points: 2.
struct AgBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        if (a.mode & MODE_STAGE_IN) BlockCopyBytes(const_cast<char*>(a.src[me]) + sb, a.in + sb, se - sb);
        RankBarrier(c, b, 0, e + 1, K_AG);
        {
            CopySeg segs[kMaxDevRanks];
            int n = 0;
            for (int k = 1; k < p; ++k) {
                const int q = (me + k) % p;
                size_t qb, qe;
                Share(a.cnt[q], nb, b, 16, &qb, &qe);
                segs[n++] = CopySeg{a.out + a.dsp[q] + qb, a.src[q] + qb, qe - qb};
            }
            if (!(a.mode & MODE_INPLACE)) BlockCopyRemoteAndLocal(segs, n, CopySeg{a.out + a.dsp[me] + sb, a.in + sb, se - sb});
            else BlockCopyMulti(segs, n);
        }
        RankBarrier(c, b, 0, e + 2, K_AG);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// AllGather LL: every rank pushes its cnt[me] (<= kLLMaxPayload) bytes as LL
// lines to all peers; one latency, no barrier.  cnt equal on all ranks.
struct AgLLBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t ep = LoadLLEpoch(c);
        const uint32_t flag = LLFlag(ep);
        const int parity = (int)(ep & 1u);
        const size_t bytes = a.cnt[me];
        const size_t nLines = (bytes + 7) >> 3;
        size_t lb, le;
        Share(nLines, nb, b, 1, &lb, &le);
        LLCreditWait(c, ep, K_AG_LL, b);
        const bool inAl = (((uintptr_t)a.in) & 7u) == 0;
        for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
            uint32_t d0, d1;
            LoadPayload8(a.in, i << 3, bytes, inAl, &d0, &d1);
            for (int k = 1; k < p; ++k) {
                const int q = (me + k) % p;
                LLStore(LLSlot(c, q, parity, me) + (i << 4), d0, d1, flag);
            }
            if (!(a.mode & MODE_INPLACE))
                StorePayload8(a.out + a.dsp[me], i << 3, bytes, (((uintptr_t)(a.out + a.dsp[me])) & 7u) == 0, d0, d1);
        }
        for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
            uint4 raw[kMaxDevRanks];
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q)
                if (q < p && q != me) raw[q] = LLPeek(LLSlot(c, me, parity, q) + (i << 4));
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q) {
                if (q < p && q != me) {
                    uint32_t d0 = raw[q].x, d1 = raw[q].z;
                    bool ok = true;
                    if (raw[q].y != flag || raw[q].w != flag)
                        ok = LLLoad(c, LLSlot(c, me, parity, q) + (i << 4), flag, &d0, &d1, K_AG_LL, b, q);
                    char* o = a.out + a.dsp[q];
                    if (ok) StorePayload8(o, i << 3, bytes, (((uintptr_t)o) & 7u) == 0, d0, d1);
                }
            }
        }
        FinishLLEpoch(c, ep, nb);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// LL exchange: the small-message form of ReduceScatter, Broadcast and AlltoAll.  Every pair moves at most `bytes`
// (<= kLLMaxPayload) as flag-in-data lines, so the op costs one NVLink latency and no barrier.
//   cnt2[q] != 0 : this rank sends `bytes` from in + dsp2[q] to rank q
//   cnt[q]  != 0 : this rank receives `bytes` from rank q; without REDUCE they land at out + dsp[q]
// With REDUCE the contributions of all ranks (this rank's own read from in + dsp2[me]) are reduced in rank order into
// out.  Without REDUCE the own block, when cnt[me] != 0, is copied locally.
template <class T, bool REDUCE>
struct LLExchangeBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        using Tr = ElemTraits<T>;
        constexpr int EPL = 8 / (int)sizeof(T) > 0 ? 8 / (int)sizeof(T) : 1;
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t ep = LoadLLEpoch(c);
        const uint32_t flag = LLFlag(ep);
        const int parity = (int)(ep & 1u);
        const size_t bytes = a.bytes;
        const size_t nLines = (bytes + 7) >> 3;
        size_t lb, le;
        Share(nLines, nb, b, 1, &lb, &le);
        LLCreditWait(c, ep, K_RS_LL, b);
        for (int k = 1; k < p; ++k) {
            const int q = (me + k) % p;
            if (a.cnt2[q] == 0) continue;
            const char* src = a.in + a.dsp2[q];
            const bool al = (((uintptr_t)src) & 7u) == 0;
            char* slot = LLSlot(c, q, parity, me);
            for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
                uint32_t d0, d1;
                LoadPayload8(src, i << 3, bytes, al, &d0, &d1);
                LLStore(slot + (i << 4), d0, d1, flag);
            }
        }
        const char* own = a.in + a.dsp2[me];
        const bool ownAl = (((uintptr_t)own) & 7u) == 0;
        for (size_t i = lb + threadIdx.x; i < le; i += blockDim.x) {
            uint4 raw[kMaxDevRanks];
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q)
                if (q < p && q != me && a.cnt[q] != 0) raw[q] = LLPeek(LLSlot(c, me, parity, q) + (i << 4));
            typename Tr::Acc acc[EPL];
            bool ok = true;
#pragma unroll
            for (int q = 0; q < kMaxDevRanks; ++q) {
                if (q >= p || a.cnt[q] == 0) continue;
                uint32_t w[2];
                if (q == me) {
                    LoadPayload8(own, i << 3, bytes, ownAl, &w[0], &w[1]);
                } else {
                    w[0] = raw[q].x;
                    w[1] = raw[q].z;
                    if (raw[q].y != flag || raw[q].w != flag)
                        ok = LLLoad(c, LLSlot(c, me, parity, q) + (i << 4), flag, &w[0], &w[1], K_RS_LL, b, q) && ok;
                }
                if (REDUCE) {
                    const T* el = reinterpret_cast<const T*>(w);
#pragma unroll
                    for (int k = 0; k < EPL; ++k) acc[k] = q == 0 ? Tr::Load(el[k]) : ApplyOp(acc[k], Tr::Load(el[k]), a.op);
                } else if (ok) {
                    char* o = a.out + a.dsp[q];
                    StorePayload8(o, i << 3, bytes, (((uintptr_t)o) & 7u) == 0, w[0], w[1]);
                }
            }
            if (REDUCE) {
                uint32_t r[2] = {0u, 0u};
                T* rl = reinterpret_cast<T*>(r);
#pragma unroll
                for (int k = 0; k < EPL; ++k) rl[k] = Tr::Store(acc[k]);
                if (ok) StorePayload8(a.out, i << 3, bytes, (((uintptr_t)a.out) & 7u) == 0, r[0], r[1]);
            }
        }
        FinishLLEpoch(c, ep, nb);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// Broadcast.  `bytes` = message; src[root] = root's (staged or symmetric) data.
// Two-shot: rank q pulls slice q from the root into out and into its exchange
// region, then every rank pulls the other slices from their owners
// (scatter + allgather, reference broadcast_mesh_1D_two_shot).  Root egress is
// ~1x the message instead of (p-1)x.  Sync points: 3.
struct BcastBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        // a block row stages exactly the bytes that the same block row of the peers reads after the barrier (rows only
        // synchronise with the same row): the one-shot form reads one contiguous share per row, the two-shot form
        // sub-range b of every slice
        if (me == root && (a.mode & MODE_STAGE_IN)) {
            if (a.mode & MODE_PUSH) {
                size_t off, end;
                Share(a.bytes, nb, b, 16, &off, &end);
                BlockCopyBytes(const_cast<char*>(a.src[root]) + off, a.in + off, end - off);
            } else {
                for (int s = 0; s < p; ++s) {
                    size_t off, len;
                    SliceSub(a.bytes, p, s, nb, b, &off, &len);
                    BlockCopyBytes(const_cast<char*>(a.src[root]) + off, a.in + off, len);
                }
            }
        }
        RankBarrier(c, b, 0, e + 1, K_BCAST);
        if (a.mode & MODE_PUSH) {
            // one-shot: every non-root pulls the whole message from the root
            if (me != root) {
                size_t off, end;
                Share(a.bytes, nb, b, 16, &off, &end);
                BlockCopyBytes(a.out + off, a.src[root] + off, end - off);
            }
            RankBarrier(c, b, 0, e + 2, K_BCAST);
            StoreEpoch(c, b, e + 2);
            OpTail(c, b);
            return;
        }
        size_t off, len;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        if (me != root) {
            BlockCopyBytes(a.xch[me] + off, a.src[root] + off, len);
            __syncthreads();
            BlockCopyBytes(a.out + off, a.xch[me] + off, len);
        }
        RankBarrier(c, b, 0, e + 2, K_BCAST);
        if (me != root) {
            CopySeg segs[kMaxDevRanks];
            int n = 0;
            for (int k = 1; k < p; ++k) {
                const int q = (me + k) % p;
                size_t qo, ql;
                SliceSub(a.bytes, p, q, nb, b, &qo, &ql);
                // the root's own slice only exists in the root's source buffer
                segs[n++] = CopySeg{a.out + qo, (q == root ? a.src[root] : a.xch[q]) + qo, ql};
            }
            BlockCopyMulti(segs, n);
        }
        RankBarrier(c, b, 0, e + 3, K_BCAST);
        StoreEpoch(c, b, e + 3);
        OpTail(c, b);
    }
};

// Broadcast through the switch: the root multimem-stores the message into the
// multicast alias of every rank's exchange region, non-roots copy it out.
struct BcastNvlsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        size_t off, end;
        Share(a.bytes, nb, b, 16, &off, &end);
        // MODE_PUSH: the buffer itself is symmetric memory with a multicast alias: the root stores straight into every
        // rank's buffer.  Otherwise the message goes through the exchange region and non-roots copy it out.
        const bool direct = (a.mode & MODE_PUSH) != 0;
        // every rank has reached the op: its buffer - or its exchange region, out of which it may still be copying the
        // result of the previous operator - may be overwritten
        RankBarrier(c, b, 0, e + 1, K_BCAST_NVLS);
        if (me == root) {
            const size_t n = end - off, nv = n >> 4;
            const bool inAl = (((uintptr_t)(a.in + off)) & 15u) == 0;
            size_t i = threadIdx.x;
            const size_t st = blockDim.x;
            if (inAl) {
                for (; i + 3 * st < nv; i += 4 * st) {
                    const uint4 v0 = LdVec(a.in + off + (i << 4)), v1 = LdVec(a.in + off + ((i + st) << 4));
                    const uint4 v2 = LdVec(a.in + off + ((i + 2 * st) << 4)), v3 = LdVec(a.in + off + ((i + 3 * st) << 4));
                    MultimemSt(a.dstMc + off + (i << 4), v0);
                    MultimemSt(a.dstMc + off + ((i + st) << 4), v1);
                    MultimemSt(a.dstMc + off + ((i + 2 * st) << 4), v2);
                    MultimemSt(a.dstMc + off + ((i + 3 * st) << 4), v3);
                }
            }
            for (; i < nv; i += st) {
                uint4 v;
                if (inAl) v = LdVec(a.in + off + (i << 4));
                else {
                    char* vb = reinterpret_cast<char*>(&v);
                    for (int k = 0; k < 16; ++k) vb[k] = a.in[off + (i << 4) + k];
                }
                MultimemSt(a.dstMc + off + (i << 4), v);
            }
            // tail (< 16 bytes): plain stores to every rank
            for (size_t t = (nv << 4) + threadIdx.x; t < n; t += blockDim.x)
                for (int q = 0; q < c.nRanks; ++q) (direct ? a.dst[q] : a.xch[q])[off + t] = a.in[off + t];
        }
        RankBarrier(c, b, 0, e + 2, K_BCAST_NVLS);
        if (!direct && me != root) BlockCopyBytes(a.out + off, a.xch[me] + off, end - off);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// Reduce to root.  Two-shot: rank q reduces slice q into its exchange region,
// the root pulls the slices (reference reduce_mesh_1D_two_shot).  One-shot
// (MODE_PUSH set): the root reduces everything itself.  Sync points: 3 / 2.
template <class T>
struct ReduceBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            // staged by the partition the readers use (see BcastBody): one contiguous share per row in the one-shot form
            if (a.mode & MODE_PUSH) {
                size_t off, end;
                Share(a.bytes, nb, b, 16, &off, &end);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, end - off);
            } else {
                for (int s = 0; s < p; ++s) {
                    size_t off, len;
                    SliceSub(a.bytes, p, s, nb, b, &off, &len);
                    BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, len);
                }
            }
        }
        RankBarrier(c, b, 0, e + 1, K_REDUCE);
        const char* srcs[kMaxDevRanks];
        if (a.mode & MODE_PUSH) {
            if (me == root) {
                size_t off, end;
                Share(a.bytes, nb, b, 16, &off, &end);
                for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + off;
                BlockReduceRange<T>(srcs, p, a.out + off, nullptr, 0, end - off, a.op);
            }
            RankBarrier(c, b, 0, e + 2, K_REDUCE);
            StoreEpoch(c, b, e + 2);
            OpTail(c, b);
            return;
        }
        size_t off, len;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + off;
        if (me == root) BlockReduceRange<T>(srcs, p, a.out + off, nullptr, 0, len, a.op);
        else BlockReduceRange<T>(srcs, p, a.xch[me] + off, nullptr, 0, len, a.op);
        RankBarrier(c, b, 0, e + 2, K_REDUCE);
        if (me == root) {
            CopySeg segs[kMaxDevRanks];
            int n = 0;
            for (int k = 1; k < p; ++k) {
                const int q = (me + k) % p;
                size_t qo, ql;
                SliceSub(a.bytes, p, q, nb, b, &qo, &ql);
                segs[n++] = CopySeg{a.out + qo, a.xch[q] + qo, ql};
            }
            BlockCopyMulti(segs, n);
        }
        RankBarrier(c, b, 0, e + 3, K_REDUCE);
        StoreEpoch(c, b, e + 3);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// Scatter: rank q pulls its block (`bytes` long) of the root's input.  The block
// of rank q sits at in + dsp2[q] in the root's user buffer and at
// src[root] + dsp[q] in the peer-visible copy.
struct ScatterBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        size_t off, end;
        Share(a.bytes, nb, b, 16, &off, &end);
        if (me == root && (a.mode & MODE_STAGE_IN)) {
            for (int q = 0; q < p; ++q)
                if (q != root)
                    BlockCopyBytes(const_cast<char*>(a.src[root]) + a.dsp[q] + off, a.in + a.dsp2[q] + off, end - off);
        }
        RankBarrier(c, b, 0, e + 1, K_SCATTER);
        if (me == root) BlockCopyBytes(a.out + off, a.in + a.dsp2[me] + off, end - off);
        else BlockCopyBytes(a.out + off, a.src[root] + a.dsp[me] + off, end - off);
        RankBarrier(c, b, 0, e + 2, K_SCATTER);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// AlltoAll / AlltoAllV / AlltoAllVC, pull form.
//   cnt[q]  = bytes this rank receives from q      dsp[q]  = where they go in `out`
//   cnt2[q] = bytes this rank sends to q           dsp2[q] = where they start in `in`
// A receiver needs the SENDER's displacement towards it, which only the sender
// knows, so every block row first publishes its rank's send displacements (and
// send sizes) in a small table inside its exchange region
// ([kMaxBlocks][2][kMaxDevRanks] uint64), and reads the peers' tables after the
// first barrier.  With MODE_STAGE_IN the send ranges are copied into the slab.
//
// Staged AlltoAllV of any size (chunk != 0): a pair's data goes through a window of
// `chunk` bytes per peer.  How many passes that takes depends on the largest
// pair of the WHOLE matrix, which no rank knows on the host (counts are private
// to each rank), so the kernel works it out: after the first barrier every
// block row reads all P x P send sizes from the tables, takes the maximum and
// loops ceil(max / window) times - the same number on every rank - where the
// window is `chunk` or, when the largest pair is smaller, that pair's size (so
// that the block rows share the bytes that actually move, not an empty window).
// Pass k moves bytes [k * window, (k + 1) * window) of every pair: stage,
// barrier, pull, barrier (nobody restages while a peer still reads).  The
// reference paces the same loop with per-peer credit flags
// (aiv_all_to_all_v_mesh_1D.h:184-214).
struct A2aSendOffsets { uint64_t v[kMaxDevRanks]; };
struct A2aBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        uint64_t* myMeta = reinterpret_cast<uint64_t*>(a.xch[me]) + (size_t)b * 2 * kMaxDevRanks;
        const bool windowed = (a.mode & MODE_STAGE_IN) && a.chunk != 0;
        const size_t win = (a.chunk + 15) & ~(size_t)15;             // distance between the peers' windows in the slab
        if (windowed) {
            // sizes first: the window split depends on the largest pair of the whole matrix
            if (threadIdx.x < p) {
                myMeta[threadIdx.x] = (uint64_t)threadIdx.x * win;
                myMeta[kMaxDevRanks + threadIdx.x] = a.cnt2[threadIdx.x];
            }
        } else if (a.mode & MODE_STAGE_IN) {
            size_t run = 0;
            for (int q = 0; q < p; ++q) {
                size_t sb, se;
                Share(a.cnt2[q], nb, b, 16, &sb, &se);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + run + sb, a.in + a.dsp2[q] + sb, se - sb);
                if (threadIdx.x == 0) myMeta[q] = run;
                run += (a.cnt2[q] + 15) & ~(size_t)15;
            }
        } else if (threadIdx.x < p) {
            myMeta[threadIdx.x] = a.dsp2[threadIdx.x];
        }
        RankBarrier(c, b, 0, e + 1, K_A2AV);
        // where each peer keeps its data for this rank: one remote read per peer, all in flight together
        HCCL_SHARED(A2aSendOffsets, s_sd);
        if ((int)threadIdx.x < p && (int)threadIdx.x != me)
            s_sd.v[threadIdx.x] = reinterpret_cast<const volatile uint64_t*>(a.xch[threadIdx.x])[(size_t)b * 2 * kMaxDevRanks + me];
        uint64_t passes = 1;
        // A block row owns the same byte range [wb, we) of every window in every pass (clipped to what the pass moves):
        // block rows only synchronise with the same row of the peers, so a row must never restage bytes that another
        // row's reader may still be pulling.  The range is a share of the EFFECTIVE window: the configured one, or the
        // largest pair when that is smaller, so that a small exchange still uses every block row.
        size_t wb = 0, we = 0, eff = 0;
        if (windowed) {
            HCCL_SHARED(unsigned long long, s_max);
            if (threadIdx.x == 0) s_max = 0ull;
            __syncthreads();
            if ((int)threadIdx.x < p * p) {
                const int q = threadIdx.x / p, r = threadIdx.x % p;
                const uint64_t v = reinterpret_cast<const volatile uint64_t*>(a.xch[q])[(size_t)b * 2 * kMaxDevRanks + kMaxDevRanks + r];
                atomicMax(&s_max, (unsigned long long)v);
            }
            __syncthreads();
            const uint64_t mx = s_max;
            eff = mx >= a.chunk ? (size_t)a.chunk : (size_t)((mx + 15) & ~(uint64_t)15);
            if (eff == 0) eff = 16;
            passes = mx == 0 ? 1 : (mx + eff - 1) / eff;
            Share(eff, nb, b, 16, &wb, &we);
        } else {
            __syncthreads();
        }
        for (uint64_t k = 0; k < passes; ++k) {
            const size_t base = windowed ? (size_t)k * eff : 0;
            if (windowed) {
                for (int q = 0; q < p; ++q) {
                    const size_t left = a.cnt2[q] > base ? a.cnt2[q] - base : 0;
                    const size_t n0 = left < eff ? left : eff;
                    const size_t sb = wb < n0 ? wb : n0, se = we < n0 ? we : n0;
                    BlockCopyBytes(const_cast<char*>(a.src[me]) + (size_t)q * win + sb, a.in + a.dsp2[q] + base + sb, se - sb);
                }
                RankBarrier(c, b, 0, e + 2 + 2 * k, K_A2AV);
            }
            {
                CopySeg segs[kMaxDevRanks];
                CopySeg own{nullptr, nullptr, 0};
                int n = 0;
                for (int kk = 0; kk < p; ++kk) {
                    const int q = (me + kk) % p;
                    size_t len = a.cnt[q];
                    if (windowed) {
                        const size_t left = a.cnt[q] > base ? a.cnt[q] - base : 0;
                        len = left < eff ? left : eff;
                    }
                    size_t rb, re;
                    if (windowed) { rb = wb < len ? wb : len; re = we < len ? we : len; }
                    else Share(len, nb, b, 16, &rb, &re);
                    if (q == me) own = CopySeg{a.out + a.dsp[q] + base + rb, a.in + a.dsp2[me] + base + rb, re - rb};
                    else segs[n++] = CopySeg{a.out + a.dsp[q] + base + rb, a.src[q] + s_sd.v[q] + rb, re - rb};
                }
                BlockCopyRemoteAndLocal(segs, n, own);
            }
            RankBarrier(c, b, 0, windowed ? e + 3 + 2 * k : e + 2, K_A2AV);
        }
        StoreEpoch(c, b, windowed ? e + 1 + 2 * passes : e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// Send / Recv / BatchSendRecv: per ordered pair (s -> d) a mailbox of two
// half-buffers lives in d's slab; sequence numbers persist in device memory so
// chunks of consecutive messages continue the same numbering (graph-replayable).
// Sender, chunk n (global numbering for the pair): wait ack >= n-1 (half free),
// write the chunk into d's mailbox half n&1, signal data = n.  Receiver: wait
// data >= n, copy out, signal ack = n.  A message that fits the two halves is
// sent without waiting for the receiver; this mirrors the staged
// ack / data / fin-ack p2p of the reference (alg_param.h:88-90) with the
// fin-ack folded into the next message's credit check.
__device__ __forceinline__ uint64_t* P2pFlag(const DevComm& c, int owner, int kind /*0 data,1 ack*/, int from)
{
    return reinterpret_cast<uint64_t*>(c.slab[owner] + kSlabP2pFlagsOff) + (size_t)kind * kMaxDevRanks + from;
}
__device__ __forceinline__ char* Mailbox(const DevComm& c, const P2pArgs& a, int owner, int from, int half)
{
    return c.slab[owner] + kSlabDataOff + a.mailboxOff + ((size_t)from * 2 + half) * a.halfBytes;
}
// One block per item (block index = item index).
struct P2pBody {
    using Args = P2pArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int)
    {
        HCCL_SHARED(int, s_ok);
        OpHead(c, b);
        if (b < a.nItems) {
            const P2pItem it = a.items[b];
            const int me = c.rank, peer = it.peer;
            const uint64_t nChunks = it.bytes == 0 ? 1 : (it.bytes + a.halfBytes - 1) / a.halfBytes;
            uint64_t* seqp = a.seq + (it.isSend ? 0 : kMaxDevRanks) + peer;
            const uint64_t first = *reinterpret_cast<volatile uint64_t*>(seqp) + 1;  // chunk numbers start at 1
            for (uint64_t k = 0; k < nChunks; ++k) {
                const uint64_t n = first + k;
                const size_t off = k * a.halfBytes;
                const size_t len = it.bytes - off < a.halfBytes ? it.bytes - off : a.halfBytes;
                __syncthreads();
                if (threadIdx.x == 0) {
                    bool ok;
                    if (it.isSend) ok = n <= 2 || WaitFlagGE(c, P2pFlag(c, me, 1, peer), n - 2, K_SENDRECV, b, 1, peer);
                    else ok = WaitFlagGE(c, P2pFlag(c, me, 0, peer), n, K_SENDRECV, b, 0, peer);
                    s_ok = ok ? 1 : 0;
                }
                __syncthreads();
                if (!s_ok) break;
                if (it.isSend) BlockCopyBytes(Mailbox(c, a, peer, me, (int)(n & 1u)), it.buf + off, len);
                else BlockCopyBytes(it.buf + off, Mailbox(c, a, me, peer, (int)(n & 1u)), len);
                __syncthreads();
                if (threadIdx.x == 0) {
                    __threadfence_system();
                    StReleaseSys(P2pFlag(c, peer, it.isSend ? 0 : 1, me), n);
                }
            }
            __syncthreads();
            if (threadIdx.x == 0) *reinterpret_cast<volatile uint64_t*>(seqp) = first + nChunks - 1;
        }
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------
// Test-only body: waits on a flag that nothing sets, to exercise the bounded
// wait and the status block (the wait must give up after timeoutNs and the
// context must stay usable).
struct TestWaitBody {
    using Args = CollArgs;
    static constexpr int kThreads = 64;
    __device__ static void Run(const DevComm& c, const Args&, int b, int)
    {
        if (threadIdx.x == 0)
            WaitFlagGE(c, FlagPtr(c, c.rank, b, kFlagSlots - 1, (c.rank + 1) % kMaxDevRanks), ~0ull, K_TEST_WAIT, b,
                       kFlagSlots - 1, (c.rank + 1) % kMaxDevRanks);
    }
};

}  // namespace hccl
