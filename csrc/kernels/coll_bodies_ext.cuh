// More kernel bodies of the collective operators:
//   * reductions fused with a data type cast and a scale (gradient averaging, fp32 -> bf16 / bf16 -> fp32 on the way),
//     the widen - reduce - narrow pattern of the reference's hif8 ReduceScatter kernel
//     (aiv_reduce_scatter_mesh_1d_hif8.h) generalised to any of fp32 / bf16 / fp16 on either side;
//   * the ring and recursive halving-doubling templates as device kernels (reference templates
//     ins_temp_reduce_scatter_ring / ins_temp_all_gather_ring, ins_temp_reduce_scatter_rhd.cc:195-238 and the
//     halving-doubling AllReduce): neighbour / partner flags instead of all-rank barriers between the steps;
//   * switch-multicast AllGather (every rank multimem-stores its block once, the switch replicates it) and Broadcast
//     as scatter + switch AllGather (reference broadcast_mesh_1D_two_shot, with the second shot through the switch);
//   * AlltoAll through the receivers' slabs: posted writes, one barrier, a local copy.
#pragma once
#include "coll_bodies.cuh"

namespace hccl {

// ---------------------------------------------------------------------------------------------------------------
// Cast + scale reductions.  T = element type of the inputs, TO = element type of the output; accumulation in fp32.
template <class TO, int N>
__device__ __forceinline__ void StoreScaled(char* dst, const float* acc, float scale, bool aligned)
{
    alignas(16) TO tmp[N];
#pragma unroll
    for (int i = 0; i < N; ++i) tmp[i] = ElemTraits<TO>::Store(acc[i] * scale);
    if (aligned) {
        constexpr int kBytes = N * (int)sizeof(TO);
        if (kBytes >= 16) {
#pragma unroll
            for (int v = 0; v < kBytes / 16; ++v) StVec(dst + v * 16, reinterpret_cast<const uint4*>(tmp)[v]);
        } else {
            *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(tmp);
        }
    } else {
        TO* d = reinterpret_cast<TO*>(dst);
#pragma unroll
        for (int i = 0; i < N; ++i) d[i] = tmp[i];
    }
}

// Reduces nElems elements from p equally aligned sources of T (16-byte aligned) into dst (elements of TO), scaled.
// One block, all threads.  U vectors of every source are requested before any is consumed.
template <class T, class TO>
__device__ __forceinline__ void BlockReduceCast(const char* const* srcs, int p, char* dst, size_t nElems, int op, float scale)
{
    constexpr int N = ElemTraits<T>::N;
    const size_t nv = nElems / N;
    const size_t nt = blockDim.x;
    const bool srcAligned = (((uintptr_t)srcs[0]) & 15u) == 0;
    const bool dstAligned = (((uintptr_t)dst) % (N * sizeof(TO) >= 16 ? 16 : N * sizeof(TO))) == 0;
    size_t done = 0;
    if (srcAligned) {
        constexpr int U = 2;
        size_t i = threadIdx.x;
        for (; i < nv; i += U * nt) {
            uint4 raw[U][kMaxDevRanks];
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int q = 0; q < kMaxDevRanks; ++q)
                    if (q < p && i + u * nt < nv) raw[u][q] = LdVec(srcs[q] + ((i + u * nt) << 4));
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (i + u * nt >= nv) continue;
                AccVec<T> acc;
                Unpack<T>(raw[u][0], acc);
#pragma unroll
                for (int q = 1; q < kMaxDevRanks; ++q)
                    if (q < p) Accumulate<T>(raw[u][q], acc, op);
                float f[N];
#pragma unroll
                for (int k = 0; k < N; ++k) f[k] = (float)acc.v[k];
                StoreScaled<TO, N>(dst + (i + u * nt) * N * sizeof(TO), f, scale, dstAligned);
            }
        }
        done = nv * N;
    }
    for (size_t e = done + threadIdx.x; e < nElems; e += nt) {
        float acc = ElemTraits<T>::Load(reinterpret_cast<const T*>(srcs[0])[e]);
        for (int q = 1; q < p; ++q) acc = ApplyOp(acc, (float)ElemTraits<T>::Load(reinterpret_cast<const T*>(srcs[q])[e]), op);
        reinterpret_cast<TO*>(dst)[e] = ElemTraits<TO>::Store(acc * scale);
    }
}

// AllReduce with cast and scale, one-shot.  bytes = input bytes of the whole message.  Sync points: 2.
template <class T, class TO>
struct ArOneShotCastBody {
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
        BlockReduceCast<T, TO>(srcs, p, a.out + off / sizeof(T) * sizeof(TO), (end - off) / sizeof(T), a.op, a.scale == 0.f ? 1.f : a.scale);
        RankBarrier(c, b, 0, e + 2, K_AR_ONESHOT);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// AllReduce with cast and scale, two-shot: rank q reduces slice q into its exchange region already as TO, then
// every rank pulls the other slices.  Sync points: 3.
template <class T, class TO>
struct ArTwoShotCastBody {
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
        const size_t oOff = off / sizeof(T) * sizeof(TO), oLen = len / sizeof(T) * sizeof(TO);
        BlockReduceCast<T, TO>(srcs, p, a.xch[me] + oOff, len / sizeof(T), a.op, a.scale == 0.f ? 1.f : a.scale);
        __syncthreads();
        BlockCopyBytes(a.out + oOff, a.xch[me] + oOff, oLen);
        RankBarrier(c, b, 0, e + 2, K_AR_TWOSHOT);
        {
            CopySeg segs[kMaxDevRanks];
            int n = 0;
            for (int k = 1; k < p; ++k) {
                const int q = (me + k) % p;
                size_t qo, ql;
                SliceSub(a.bytes, p, q, nb, b, &qo, &ql);
                segs[n++] = CopySeg{a.out + qo / sizeof(T) * sizeof(TO), a.xch[q] + qo / sizeof(T) * sizeof(TO), ql / sizeof(T) * sizeof(TO)};
            }
            BlockCopyMulti(segs, n);
        }
        RankBarrier(c, b, 0, e + 3, K_AR_TWOSHOT);
        StoreEpoch(c, b, e + 3);
        OpTail(c, b);
    }
};

// ReduceScatter with cast and scale: cnt / dsp / dsp2 in INPUT bytes as in RsBody.  Sync points: 2.
template <class T, class TO>
struct RsCastBody {
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
        RankBarrier(c, b, 0, e + 1, K_RS);
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        const char* srcs[kMaxDevRanks];
        for (int q = 0; q < p; ++q) srcs[q] = a.src[q] + a.dsp[me] + sb;
        BlockReduceCast<T, TO>(srcs, p, a.out + sb / sizeof(T) * sizeof(TO), (se - sb) / sizeof(T), a.op, a.scale == 0.f ? 1.f : a.scale);
        RankBarrier(c, b, 0, e + 2, K_RS);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// Ring and halving-doubling templates.  Steps are ordered by one-directional flags between the two ranks involved
// (flag slot kStepSlot of the block row); the value of step s of an operator that started at epoch e is
// (e + 1) * 16 + s, which only grows from operator to operator.  Partial results travel through per-step slots of the
// exchange region, so nothing is overwritten inside an operator; the closing barrier keeps the next operator from
// overwriting a slot a neighbour still reads.
constexpr int kStepSlot = 2;
__device__ __forceinline__ uint64_t StepValue(uint64_t e, int s) { return (e + 1) * 16 + (uint64_t)s; }
// all threads of the block call both; data written before SignalStep is visible after the matching WaitStep
__device__ __forceinline__ void SignalStep(const DevComm& c, int peer, int b, uint64_t value)
{
    __syncthreads();
    if (threadIdx.x == 0) SignalPeer(c, peer, b, kStepSlot, value);
}
__device__ __forceinline__ bool WaitStep(const DevComm& c, int peer, int b, uint64_t value, uint32_t kernelId)
{
    HCCL_SHARED(int, s_stepOk);
    if (threadIdx.x == 0) s_stepOk = WaitPeer(c, peer, b, kStepSlot, value, kernelId) ? 1 : 0;
    __syncthreads();
    const bool ok = s_stepOk != 0;
    __syncthreads();
    return ok;
}

// ReduceScatter on a ring.  The partial sum of block k starts at rank k + 1 and travels k + 1 -> k + 2 -> ... -> k;
// in step s (1 .. p - 1) a rank adds its own block (me - 1 - s) to the partial it reads from its left neighbour
// (the neighbour's input in step 1, its exchange slot s - 1 afterwards) and leaves the result in its own slot s, or
// in `out` in the last step.  cnt / dsp / dsp2 as in RsBody with equal cnt; slot s of the exchange region starts at
// s * bytes (bytes = 16-byte aligned block size).  Sync points: 2 barriers + p - 2 neighbour flags.
template <class T>
struct RsRingBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const int left = (me + p - 1) % p, right = (me + 1) % p;
        const uint64_t e = LoadEpoch(c, b);
        if (a.mode & MODE_STAGE_IN) {
            for (int q = 0; q < p; ++q) {
                size_t sb, se;
                Share(a.cnt[q], nb, b, 16, &sb, &se);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + a.dsp[q] + sb, a.in + a.dsp2[q] + sb, se - sb);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_RS);
        const size_t slot = (a.bytes + 15) & ~(size_t)15;
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);      // equal blocks: the same sub-range of every block
        bool ok = true;
        for (int s = 1; s < p && ok; ++s) {
            const int k = (me - 1 - s + 2 * p) % p;                       // block handled in this step
            const char* srcs[2];
            if (s == 1) {
                srcs[0] = a.src[left] + a.dsp[k] + sb;                    // the left neighbour's own block k
            } else {
                ok = WaitStep(c, left, b, StepValue(e, s - 1), K_RS);     // its partial of step s - 1 is complete
                if (!ok) break;
                srcs[0] = a.xch[left] + (size_t)(s - 1) * slot + sb;
            }
            srcs[1] = a.src[me] + a.dsp[k] + sb;
            char* dst = s == p - 1 ? a.out + sb : a.xch[me] + (size_t)s * slot + sb;
            BlockReduceRange<T>(srcs, 2, dst, nullptr, 0, se - sb, a.op);
            if (s < p - 1) SignalStep(c, right, b, StepValue(e, s));
        }
        RankBarrier(c, b, 0, e + 2, K_RS);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// AllGather on a ring: in step s a rank copies block (me - s) from its left neighbour (the neighbour's input in
// step 1, the neighbour's exchange slot afterwards) into `out` and, while a right neighbour still needs it, into its
// own exchange slot.  Equal blocks of `bytes`.  Sync points: 2 barriers + p - 2 neighbour flags.
struct AgRingBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const int left = (me + p - 1) % p, right = (me + 1) % p;
        const uint64_t e = LoadEpoch(c, b);
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        if (a.mode & MODE_STAGE_IN) BlockCopyBytes(const_cast<char*>(a.src[me]) + sb, a.in + sb, se - sb);
        RankBarrier(c, b, 0, e + 1, K_AG);
        if (!(a.mode & MODE_INPLACE)) BlockCopyBytes(a.out + a.dsp[me] + sb, a.in + sb, se - sb);
        const size_t slot = (a.bytes + 15) & ~(size_t)15;
        bool ok = true;
        for (int s = 1; s < p && ok; ++s) {
            const int k = (me - s + p) % p;
            const char* src;
            if (s == 1) {
                src = a.src[left] + sb;
            } else {
                ok = WaitStep(c, left, b, StepValue(e, s - 1), K_AG);
                if (!ok) break;
                src = a.xch[left] + (size_t)(s - 1) * slot + sb;
            }
            if (s < p - 1) {
                BlockCopyBytes(a.xch[me] + (size_t)s * slot + sb, src, se - sb);
                __syncthreads();
                BlockCopyBytes(a.out + a.dsp[k] + sb, a.xch[me] + (size_t)s * slot + sb, se - sb);
                SignalStep(c, right, b, StepValue(e, s));
            } else {
                BlockCopyBytes(a.out + a.dsp[k] + sb, src, se - sb);
            }
        }
        RankBarrier(c, b, 0, e + 2, K_AG);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// AllReduce by recursive halving (reduce-scatter) and recursive doubling (all-gather); power-of-two rank counts.
// The working copy W of the message lives in the exchange region.  Halving step k (distance d = p / 2^(k+1)): a
// rank keeps the half of its current range that contains its own final piece, reads the partner's copy of that
// half (the partner's input in step 0, its W afterwards), adds its own and writes W.  Doubling runs the steps
// backwards: a rank copies the range its partner owns from the partner's W into its own W.  A rank never rewrites
// a part of W that a partner of an earlier step may still be reading (it only writes inside the half it kept), so
// one flag per step and direction suffices.  Sync points: 2 barriers + 2 log2(p) partner flags.
template <class T>
struct ArRhdBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        // The message is cut in p pieces (piece j ends up reduced on rank j) and block row b owns sub-range b of EVERY
        // piece, in every step: rows only synchronise with the same row of the partner, so a row must only ever read
        // bytes that the same row wrote.
        if (a.mode & MODE_STAGE_IN) {
            for (int j = 0; j < p; ++j) {
                size_t off, len;
                SliceSub(a.bytes, p, j, nb, b, &off, &len);
                BlockCopyBytes(const_cast<char*>(a.src[me]) + off, a.in + off, len);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_AR_TWOSHOT);
        int steps = 0;
        while ((1 << steps) < p) ++steps;
        int first = 0, count = p;           // pieces this rank's W currently covers
        bool ok = true;
        int sig = 0;
        for (int k = 0; k < steps && ok; ++k) {
            const int half = count / 2;
            const int partner = me ^ half;
            const int kFirst = (me & half) == 0 ? first : first + half;
            if (k > 0) {
                ok = WaitStep(c, partner, b, StepValue(e, sig), K_AR_TWOSHOT);   // the partner finished halving step k - 1
                if (!ok) break;
            }
            for (int j = kFirst; j < kFirst + half; ++j) {
                size_t off, len;
                SliceSub(a.bytes, p, j, nb, b, &off, &len);
                const char* srcs[2];
                srcs[0] = (k == 0 ? a.src[partner] : a.xch[partner]) + off;
                srcs[1] = (k == 0 ? a.src[me] : a.xch[me]) + off;
                BlockReduceRange<T>(srcs, 2, a.xch[me] + off, nullptr, 0, len, a.op);
            }
            first = kFirst;
            count = half;
            ++sig;
            if (k + 1 < steps) SignalStep(c, me ^ (count / 2), b, StepValue(e, sig));
        }
        // W[piece me] is final: hand it to `out`, then double
        __syncthreads();
        {
            size_t off, len;
            SliceSub(a.bytes, p, first, nb, b, &off, &len);
            BlockCopyBytes(a.out + off, a.xch[me] + off, len);
        }
        for (int k = steps - 1; k >= 0 && ok; --k) {
            const int partner = me ^ count;             // count = pieces held so far = distance of this doubling step
            ++sig;
            SignalStep(c, partner, b, StepValue(e, sig));                        // my `count` pieces are complete in W
            ok = WaitStep(c, partner, b, StepValue(e, sig), K_AR_TWOSHOT);
            if (!ok) break;
            const int pFirst = (me & count) ? first - count : first + count;
            for (int j = pFirst; j < pFirst + count; ++j) {
                size_t off, len;
                SliceSub(a.bytes, p, j, nb, b, &off, &len);
                BlockCopyBytes(a.xch[me] + off, a.xch[partner] + off, len);
            }
            __syncthreads();
            for (int j = pFirst; j < pFirst + count; ++j) {
                size_t off, len;
                SliceSub(a.bytes, p, j, nb, b, &off, &len);
                BlockCopyBytes(a.out + off, a.xch[me] + off, len);
            }
            first = first < pFirst ? first : pFirst;
            count *= 2;
        }
        RankBarrier(c, b, 0, e + 2, K_AR_TWOSHOT);
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// AllGather through the switch: every rank multimem-stores its block into the multicast alias of the destination
// (dstMc + dsp2[me]); its NVLink port carries the block once instead of p - 1 times.  dst is either the output
// itself (symmetric memory with a multicast alias, MODE_PUSH, dsp2 = dsp) or the exchange region (blocks packed at
// dsp2), from which every rank copies the gathered data out to out + dsp.  Equal 16-byte aligned blocks.  Sync points: 2.  Remote writes into an exchange region only
// ever start after an all-rank barrier inside the same operator, because some operators read their results out of
// that region after their last barrier.
struct AgNvlsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        const bool direct = (a.mode & MODE_PUSH) != 0;
        size_t sb, se;
        Share(a.cnt[me], nb, b, 16, &sb, &se);
        // every rank is inside the operator: the destination (a user buffer, or the exchange region that a peer may still
        // be copying the previous operator's result out of) may be overwritten
        RankBarrier(c, b, 0, e + 1, K_AG_NVLS);
        {
            const size_t n = se - sb, nv = n >> 4;
            const char* in = a.in + sb;
            char* mc = a.dstMc + a.dsp2[me] + sb;
            const bool inAl = (((uintptr_t)in) & 15u) == 0;
            const size_t st = blockDim.x;
            size_t i = threadIdx.x;
            if (inAl) {
                for (; i + 3 * st < nv; i += 4 * st) {
                    uint4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) v[u] = LdVec(in + ((i + u * st) << 4));
#pragma unroll
                    for (int u = 0; u < 4; ++u) MultimemSt(mc + ((i + u * st) << 4), v[u]);
                }
            }
            for (; i < nv; i += st) {
                uint4 v;
                if (inAl) v = LdVec(in + (i << 4));
                else {
                    char* vb = reinterpret_cast<char*>(&v);
                    for (int k = 0; k < 16; ++k) vb[k] = in[(i << 4) + k];
                }
                MultimemSt(mc + (i << 4), v);
            }
            for (size_t t = (nv << 4) + threadIdx.x; t < n; t += blockDim.x)
                for (int q = 0; q < p; ++q) a.dst[q][a.dsp2[me] + sb + t] = in[t];
        }
        RankBarrier(c, b, 0, e + 2, K_AG_NVLS);
        if (!direct) {
            // local copy out of the exchange region; the next operator that writes there opens with a barrier
            for (int q = 0; q < p; ++q) {
                size_t qb, qe;
                Share(a.cnt[q], nb, b, 16, &qb, &qe);
                BlockCopyBytes(a.out + a.dsp[q] + qb, a.dst[me] + a.dsp2[q] + qb, qe - qb);
            }
        }
        StoreEpoch(c, b, e + 2);
        OpTail(c, b);
    }
};

// Broadcast as scatter + switch AllGather: rank q pulls slice q of the root's data and multimem-stores it to every
// rank, so the root's port carries the message once and every other port 1 / p of it (a single sender's multicast
// stream saturates far below the port rate; p senders do not).  dst as in AgNvlsBody.  Sync points: 2.
struct BcastScatterNvlsBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        const bool direct = (a.mode & MODE_PUSH) != 0;
        if (me == root && (a.mode & MODE_STAGE_IN)) {
            for (int s = 0; s < p; ++s) {
                size_t off, len;
                SliceSub(a.bytes, p, s, nb, b, &off, &len);
                BlockCopyBytes(const_cast<char*>(a.src[root]) + off, a.in + off, len);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_BCAST_NVLS);       // the root's data is readable; every destination may be written
        size_t off, len;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        {
            const char* src = (me == root ? a.in : a.src[root]) + off;
            const size_t nv = len >> 4;
            const bool al = (((uintptr_t)src) & 15u) == 0;
            const size_t st = blockDim.x;
            size_t i = threadIdx.x;
            if (al) {
                for (; i + 7 * st < nv; i += 8 * st) {
                    uint4 v[8];
#pragma unroll
                    for (int u = 0; u < 8; ++u) v[u] = LdVec(src + ((i + u * st) << 4));
#pragma unroll
                    for (int u = 0; u < 8; ++u) MultimemSt(a.dstMc + off + ((i + u * st) << 4), v[u]);
                }
            }
            for (; i < nv; i += st) {
                uint4 v;
                if (al) v = LdVec(src + (i << 4));
                else {
                    char* vb = reinterpret_cast<char*>(&v);
                    for (int k = 0; k < 16; ++k) vb[k] = src[(i << 4) + k];
                }
                MultimemSt(a.dstMc + off + (i << 4), v);
            }
            for (size_t t = (nv << 4) + threadIdx.x; t < len; t += blockDim.x)
                for (int q = 0; q < p; ++q) a.dst[q][off + t] = src[t];
        }
        RankBarrier(c, b, 0, e + 2, K_BCAST_NVLS);
        if (!direct && me != root) {
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

// ---------------------------------------------------------------------------------------------------------------
// Broadcast of large messages as a pipelined scatter + AllGather over plain peer reads.  The message is cut into
// p - 1 slices, one per non-root rank.  In step i a rank pulls piece i of ITS slice from the root and, in the same
// pass, piece i - 1 of every other slice from the rank that pulled it one step earlier; one barrier closes a step.
// Every byte leaves the root once and enters every other rank once, and both directions of every port are busy in
// every step but the first and the last (the two-shot form runs the two phases one after the other, and a single
// multicast sender saturates far below the port rate).  `chunk` = bytes of one piece, cnt2[0] = number of pieces
// (the same on every rank); src[root] = the root's data where the peers can read it; the owners' pieces are read
// from dst[q] (MODE_PUSH: the output buffers themselves are peer-visible) or from xch[q].  Sync points: pieces + 2.
struct BcastPipeBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    // piece i of the sub-range [off, off + len)
    __device__ static void Piece(size_t len, size_t piece, int i, size_t* b0, size_t* b1)
    {
        const size_t lo = (size_t)i * piece, hi = lo + piece;
        *b0 = lo < len ? lo : len;
        *b1 = hi < len ? hi : len;
    }
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank, root = a.root;
        const uint64_t e = LoadEpoch(c, b);
        const int slices = p - 1, pieces = (int)a.cnt2[0];
        const bool direct = (a.mode & MODE_PUSH) != 0;
        const int mine = (me - root - 1 + p) % p;                 // this rank's slice (meaningless on the root)
        if (me == root && (a.mode & MODE_STAGE_IN)) {
            for (int s = 0; s < slices; ++s) {
                size_t off, len;
                SliceSub(a.bytes, slices, s, nb, b, &off, &len);
                BlockCopyBytes(const_cast<char*>(a.src[root]) + off, a.in + off, len);
            }
        }
        RankBarrier(c, b, 0, e + 1, K_BCAST);
        for (int i = 0; i <= pieces; ++i) {
            if (me != root) {
                CopySeg segs[kMaxDevRanks + 1];
                int n = 0;
                if (i < pieces) {
                    size_t off, len, b0, b1;
                    SliceSub(a.bytes, slices, mine, nb, b, &off, &len);
                    Piece(len, (size_t)a.chunk, i, &b0, &b1);
                    char* hold = direct ? a.out : a.xch[me];
                    if (b1 > b0) segs[n++] = CopySeg{hold + off + b0, a.src[root] + off + b0, b1 - b0};
                }
                if (i >= 1) {
                    for (int k = 0; k < p; ++k) {
                        const int q = (me + k) % p;
                        if (q == root || (q == me && direct)) continue;
                        const int sq = (q - root - 1 + p) % p;
                        size_t off, len, b0, b1;
                        SliceSub(a.bytes, slices, sq, nb, b, &off, &len);
                        Piece(len, (size_t)a.chunk, i - 1, &b0, &b1);
                        const char* from = direct ? a.dst[q] : a.xch[q];       // q == me: the piece this rank pulled one step ago
                        if (b1 > b0) segs[n++] = CopySeg{a.out + off + b0, from + off + b0, b1 - b0};
                    }
                }
                BlockCopyMulti(segs, n);
            }
            RankBarrier(c, b, 0, e + 2 + (uint64_t)i, K_BCAST);
        }
        StoreEpoch(c, b, e + 2 + (uint64_t)pieces);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// AlltoAll through the receivers' slabs.  The pull form pays a table exchange and two barriers around the
// transfer; here a rank WRITES its block for q into q's stage-in region (posted stores, no round trip), one
// barrier publishes everything, and every rank copies its received blocks out locally.  The landing zone holds two
// copies, taken in turn by the communicator's count of push operators (LoadPushSeq): to write for push operator
// n + 2 a rank has finished n + 1, which the peer entered after finishing n, so the copy a peer still reads is never
// the one being written.  The
// stage-in region is the one part of a slab that no other operator writes from a remote rank (its owner stages
// into it before a barrier), which is what makes the missing closing barrier safe.  `bytes` = one pair's block (equal
// for all pairs); the copy of parity h starts at src[q] + h * chunk, the block from rank r inside it at r * slot.
// Sync points: 1.
struct A2aPushBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        const size_t slot = (a.bytes + 15) & ~(size_t)15;
        const uint64_t seq = LoadPushSeq(c);
        const size_t region = (size_t)(seq & 1u) * a.chunk;
        size_t sb, se;
        Share(a.bytes, nb, b, 16, &sb, &se);
        for (int k = 1; k < p; ++k) {
            const int q = (me + k) % p;
            BlockCopyBytes(const_cast<char*>(a.src[q]) + region + (size_t)me * slot + sb, a.in + a.dsp2[q] + sb, se - sb);
        }
        BlockCopyBytes(a.out + a.dsp[me] + sb, a.in + a.dsp2[me] + sb, se - sb);
        RankBarrier(c, b, 0, e + 1, K_A2A);
        for (int k = 1; k < p; ++k) {
            const int q = (me + k) % p;
            BlockCopyBytes(a.out + a.dsp[q] + sb, a.src[me] + region + (size_t)q * slot + sb, se - sb);
        }
        StoreEpoch(c, b, e + 1);
        FinishPushSeq(c, seq, nb);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// AlltoAllV with a leader row.  The counts of an AlltoAllV are private to each rank, so the host cannot size the grid
// by the data: every rank launches the full grid, and in A2aBody every one of its (up to 128) block rows runs the
// size exchange and two barriers with its peers - 65-78 us for any exchange below a few MiB at 8 ranks where NCCL
// takes 46-50 us.  Here only block row 0 exchanges the sizes: it publishes this rank's send sizes and offsets, runs one
// barrier, reads all p x p sizes, and tells the other rows of ITS OWN rank the largest pair through two local words
// (a release store of the operator's tag after the size; the rows wait for the tag with a bounded acquire spin).
// From the largest pair every rank derives the same number of rows that take part, R = one row per 32 KiB a rank
// receives; rows >= R leave at once, without a barrier (their epochs do not move), rows < R share the data R ways and
// run the barriers the transfer itself needs (staging / closing) with the same rows of the peers.  A row b > 0 may
// read a peer's buffers without a barrier of its own: row 0 of its rank has passed the start barrier, so every peer
// is inside this operator and its tables are published, and the tag's acquire makes that visible to the row.
// Fields as in A2aBody; staged inputs always go through windows (chunk != 0).  Sync points: 2 + passes on the rows
// that take part, none on the others.
struct A2avLeaderBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    static constexpr uint64_t kBytesPerRow = 32u << 10;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t seq = LoadA2avSeq(c), tag = seq + 1;
        uint64_t ev = LoadEpoch(c, b);
        uint64_t* myMeta = reinterpret_cast<uint64_t*>(a.xch[me]);                 // row 0's table: the only one in use
        const bool staged = (a.mode & MODE_STAGE_IN) != 0;
        const size_t win = (a.chunk + 15) & ~(size_t)15;
        uint64_t* tagWord = c.epochs + kA2avTagWord;
        volatile uint64_t* maxWord = c.epochs + kA2avMaxWord;
        HCCL_SHARED(unsigned long long, s_max);
        if (b == 0) {
            if ((int)threadIdx.x < p) {
                myMeta[threadIdx.x] = staged ? (uint64_t)threadIdx.x * win : a.dsp2[threadIdx.x];
                myMeta[kMaxDevRanks + threadIdx.x] = a.cnt2[threadIdx.x];
            }
            if (threadIdx.x == 0) s_max = 0ull;
            RankBarrier(c, 0, 0, ++ev, K_A2AV);
            if ((int)threadIdx.x < p * p) {
                const int q = threadIdx.x / p, r = threadIdx.x % p;
                const uint64_t v = reinterpret_cast<const volatile uint64_t*>(a.xch[q])[kMaxDevRanks + r];
                atomicMax(&s_max, (unsigned long long)v);
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                *maxWord = (uint64_t)s_max;
                StReleaseSys(tagWord, tag);          // after the size; a failed barrier has raised the abort word already
            }
        } else {
            if (threadIdx.x == 0) {
                WaitFlagGE(c, tagWord, tag, K_A2AV, b, 0, me);
                s_max = (unsigned long long)*maxWord;
            }
            __syncthreads();
        }
        const uint64_t mx = s_max;
        uint64_t rows = (mx * (uint64_t)(p - 1) + kBytesPerRow - 1) / kBytesPerRow;
        if (rows < 1) rows = 1;
        if (rows > (uint64_t)nb) rows = (uint64_t)nb;
        const int R = (int)rows;
        if (b >= R) {
            FinishA2avSeq(c, seq, nb);
            OpTail(c, b);
            return;
        }
        // where each peer keeps its data for this rank: one remote read per peer, all in flight together
        HCCL_SHARED(A2aSendOffsets, s_sd);
        if ((int)threadIdx.x < p && (int)threadIdx.x != me) s_sd.v[threadIdx.x] = reinterpret_cast<const volatile uint64_t*>(a.xch[threadIdx.x])[me];
        __syncthreads();
        size_t eff = 0, wb = 0, we = 0;
        uint64_t passes = 1;
        if (staged) {
            eff = mx >= a.chunk ? (size_t)a.chunk : (size_t)((mx + 15) & ~(uint64_t)15);
            if (eff == 0) eff = 16;
            passes = mx == 0 ? 1 : (mx + eff - 1) / eff;
            Share(eff, R, b, 16, &wb, &we);
        }
        for (uint64_t k = 0; k < passes; ++k) {
            const size_t base = staged ? (size_t)k * eff : 0;
            if (staged) {
                for (int q = 0; q < p; ++q) {
                    const size_t left = a.cnt2[q] > base ? a.cnt2[q] - base : 0;
                    const size_t n0 = left < eff ? left : eff;
                    const size_t sb = wb < n0 ? wb : n0, se = we < n0 ? we : n0;
                    BlockCopyBytes(const_cast<char*>(a.src[me]) + (size_t)q * win + sb, a.in + a.dsp2[q] + base + sb, se - sb);
                }
                RankBarrier(c, b, 0, ++ev, K_A2AV);
            }
            CopySeg segs[kMaxDevRanks];
            CopySeg own{nullptr, nullptr, 0};
            int n = 0;
            for (int kk = 0; kk < p; ++kk) {
                const int q = (me + kk) % p;
                size_t len = a.cnt[q];
                size_t rb, re;
                if (staged) {
                    const size_t left = a.cnt[q] > base ? a.cnt[q] - base : 0;
                    len = left < eff ? left : eff;
                    rb = wb < len ? wb : len;
                    re = we < len ? we : len;
                } else {
                    Share(len, R, b, 16, &rb, &re);
                }
                if (q == me) own = CopySeg{a.out + a.dsp[q] + base + rb, a.in + a.dsp2[me] + base + rb, re - rb};
                else segs[n++] = CopySeg{a.out + a.dsp[q] + base + rb, a.src[q] + s_sd.v[q] + rb, re - rb};
            }
            BlockCopyRemoteAndLocal(segs, n, own);
            RankBarrier(c, b, 0, ++ev, K_A2AV);          // nobody restages, overwrites its buffer or leaves while a peer still reads
        }
        StoreEpoch(c, b, ev);
        FinishA2avSeq(c, seq, nb);
        OpTail(c, b);
    }
};

// ---------------------------------------------------------------------------------------------------------------
// ReduceScatter and AllReduce for ORDINARY (unregistered) buffers without the stage-in pass.  The pull forms first
// copy the whole input into the slab so that the peers can read it: a full extra pass over the message.  Here a
// rank writes block q of its input straight into rank q's slab (posted stores over NVLink, the input is read once,
// locally), one barrier publishes everything, and every rank reduces the p - 1 blocks that landed in its own slab
// with its own block, which it reads in place.  Landing zone and parity rule are those of A2aPushBody (stage-in
// region, two copies taken in turn, no closing barrier).  cnt / dsp2 as in RsBody with equal blocks of `bytes`
// (one chunk of a larger message per launch); chunk = size of one landing copy.  Sync points: 1.
template <class T>
struct RsPushBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        const size_t slot = (a.bytes + 15) & ~(size_t)15;
        const uint64_t seq = LoadPushSeq(c);
        const size_t region = (size_t)(seq & 1u) * a.chunk;
        size_t sb, se;
        Share(a.bytes, nb, b, 16, &sb, &se);
        // BlockReduceRange wants all sources equally aligned: the landed blocks are 16-byte aligned, so an input block
        // that is not goes through this rank's own landing slot as well (a local copy)
        const bool ownDirect = (((uintptr_t)(a.in + a.dsp2[me])) & 15u) == 0;
        for (int k = ownDirect ? 1 : 0; k < p; ++k) {
            const int q = (me + k) % p;
            BlockCopyBytes(const_cast<char*>(a.src[q]) + region + (size_t)me * slot + sb, a.in + a.dsp2[q] + sb, se - sb);
        }
        RankBarrier(c, b, 0, e + 1, K_RS);
        const char* srcs[kMaxDevRanks];
        for (int q = 0; q < p; ++q) srcs[q] = (q == me && ownDirect) ? a.in + a.dsp2[me] + sb : a.src[me] + region + (size_t)q * slot + sb;
        BlockReduceRange<T>(srcs, p, a.out + sb, nullptr, 0, se - sb, a.op);
        StoreEpoch(c, b, e + 1);
        FinishPushSeq(c, seq, nb);
        OpTail(c, b);
    }
};

// AllReduce for ordinary buffers, two-shot without the stage-in pass: the ReduceScatter above leaves slice `me`
// reduced in this rank's exchange region (and in `out`), then every rank pulls the other slices from their owners.
// bytes = the whole message of this launch, sliced over the ranks in 16-byte units; chunk = one landing copy.
// Sync points: 3 (landing, slices ready, slices read).
template <class T>
struct ArPushTwoShotBody {
    using Args = CollArgs;
    static constexpr int kThreads = 512;
    __device__ static void Run(const DevComm& c, const Args& a, int b, int nb)
    {
        OpHead(c, b);
        const int p = c.nRanks, me = c.rank;
        const uint64_t e = LoadEpoch(c, b);
        size_t s0, s1;
        Share(a.bytes, p, 0, 16, &s0, &s1);
        const size_t slot = s1 - s0;                               // the widest slice (slices are equal except the last)
        // the landing copies are taken in turn: a push operator without a closing barrier may have used the other one
        // just before, and its reader may still be busy
        const uint64_t seq = LoadPushSeq(c);
        const size_t region = (size_t)(seq & 1u) * a.chunk;
        const bool ownDirect = (((uintptr_t)a.in) & 15u) == 0;
        for (int k = ownDirect ? 1 : 0; k < p; ++k) {
            const int q = (me + k) % p;
            size_t off, len;
            SliceSub(a.bytes, p, q, nb, b, &off, &len);
            size_t q0, q1;
            Share(a.bytes, p, q, 16, &q0, &q1);
            BlockCopyBytes(const_cast<char*>(a.src[q]) + region + (size_t)me * slot + (off - q0), a.in + off, len);
        }
        RankBarrier(c, b, 0, e + 1, K_AR_TWOSHOT);
        size_t off, len, m0, m1;
        SliceSub(a.bytes, p, me, nb, b, &off, &len);
        Share(a.bytes, p, me, 16, &m0, &m1);
        {
            const char* srcs[kMaxDevRanks];
            for (int q = 0; q < p; ++q) srcs[q] = (q == me && ownDirect) ? a.in + off : a.src[me] + region + (size_t)q * slot + (off - m0);
            BlockReduceRange<T>(srcs, p, a.xch[me] + off, nullptr, 0, len, a.op);
            __syncthreads();
            BlockCopyBytes(a.out + off, a.xch[me] + off, len);
        }
        RankBarrier(c, b, 0, e + 2, K_AR_TWOSHOT);
        {
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
        RankBarrier(c, b, 0, e + 3, K_AR_TWOSHOT);
        StoreEpoch(c, b, e + 3);
        FinishPushSeq(c, seq, nb);
        OpTail(c, b);
    }
};

}  // namespace hccl
