// Runs the collective kernel bodies on the CPU: every CUDA thread is a host thread, every rank's slab is host memory
// in one address space, flags are atomics with the PTX's memory order, data accesses are plain (see
// csrc/kernels/host_shim.h).  Built with -fsanitize=thread it is the race detector of the flag protocols; built
// with -fsanitize=address it checks bounds.  Every operator runs twice in a row (epochs continue, line slots are
// reused) at 2, 3 and 8 ranks and is compared with a reference computed on the host.
//
//   g++ -std=c++17 -O1 -g -fsanitize=thread -DHCCL_HOST_SHIM -Icsrc -Icsrc/include -I$CUDA_HOME/include \
//       tests/cpu_harness/kernel_harness.cc -o build/kernel_harness_tsan -pthread && build/kernel_harness_tsan
#ifndef HCCL_HOST_SHIM
#define HCCL_HOST_SHIM 1
#endif
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <memory>
#include <string>
#include <thread>
#include "kernels/coll_bodies.cuh"
#include "kernels/coll_bodies_ext.cuh"

using namespace hccl;

namespace {

constexpr size_t kDataBytes = 4u << 20;          // staging data region per rank
constexpr size_t kInBytes = 1u << 20, kXchOff = 2u << 20, kXchBytes = 1u << 20, kMailboxOff = 3u << 20, kMailboxHalf = 32u << 10;

struct Rank {
    DevComm comm;
    char* slab = nullptr;
    uint64_t* epochs = nullptr;
    uint32_t* abortWord = nullptr;
    DevStatus* status = nullptr;
    uint64_t* p2pSeq = nullptr;
};

struct World {
    int p;
    std::vector<Rank> ranks;
    char* mcBase = nullptr;          // never dereferenced: stands for "the same offset in every rank's slab"
    explicit World(int n) : p(n), ranks((size_t)n)
    {
        const size_t slabBytes = kSlabDataOff + kDataBytes;
        mcBase = (char*)aligned_alloc(4096, slabBytes);
        hostshim::McWindow w{mcBase, slabBytes, {}};
        for (int r = 0; r < p; ++r) {
            Rank& k = ranks[(size_t)r];
            k.slab = (char*)aligned_alloc(4096, slabBytes);
            memset(k.slab, 0, slabBytes);
            k.epochs = (uint64_t*)calloc(kEpochWords, sizeof(uint64_t));
            k.abortWord = (uint32_t*)calloc(64, 4);
            k.status = (DevStatus*)calloc(1, sizeof(DevStatus));
            k.p2pSeq = (uint64_t*)calloc(2 * kMaxDevRanks, sizeof(uint64_t));
            w.targets.push_back(k.slab);
        }
        for (int r = 0; r < p; ++r) {
            DevComm& c = ranks[(size_t)r].comm;
            memset(&c, 0, sizeof(c));
            c.rank = r;
            c.nRanks = p;
            for (int q = 0; q < p; ++q) c.slab[q] = ranks[(size_t)q].slab;
            c.slabMc = mcBase;
            c.epochs = ranks[(size_t)r].epochs;
            c.abortWord = ranks[(size_t)r].abortWord;
            c.status = ranks[(size_t)r].status;
            c.timeoutNs = 60ull * 1000 * 1000 * 1000;
            c.stageBytes = kDataBytes;
        }
        hostshim::McWindows().clear();
        hostshim::McWindows().push_back(w);
    }
    ~World()
    {
        for (Rank& k : ranks) { free(k.slab); free(k.epochs); free(k.abortWord); free(k.status); free(k.p2pSeq); }
        free(mcBase);
        hostshim::McWindows().clear();
    }
    char* stageIn(int r) const { return ranks[(size_t)r].slab + kSlabDataOff; }
    char* xch(int r) const { return ranks[(size_t)r].slab + kSlabDataOff + kXchOff; }
    bool failed() const
    {
        for (const Rank& k : ranks)
            if (k.status->error != DEV_OK) {
                fprintf(stderr, "  rank %u: kernel family %u block %u gave up on flag slot %u of rank %u (expected %llu, saw %llu)\n", k.status->rank,
                        k.status->kernelId, k.status->block, k.status->slot, k.status->peer, (unsigned long long)k.status->expected,
                        (unsigned long long)k.status->seen);
                return true;
            }
        return false;
    }
};

// One "launch": nb blocks of `threads` threads for every rank, all running together (what a cooperative grid over all
// ranks gives on one GPU, or one kernel per GPU on a real box).
template <class Body>
void Launch(World& w, const std::vector<typename Body::Args>& args, int nb, int threads)
{
    std::vector<hostshim::BlockCtx*> blocks;
    std::vector<std::thread> pool;
    for (int r = 0; r < w.p; ++r) {
        for (int b = 0; b < nb; ++b) {
            hostshim::BlockCtx* ctx = new hostshim::BlockCtx();
            memset(ctx->shared, 0, sizeof(ctx->shared));
            pthread_barrier_init(&ctx->bar, nullptr, (unsigned)threads);
            blocks.push_back(ctx);
            for (int t = 0; t < threads; ++t) {
                pool.emplace_back([&w, &args, ctx, r, b, t, nb, threads] {
                    hostshim::ThreadCtx& me = hostshim::Tls();
                    me.tid.x = (unsigned)t;
                    me.bid.x = (unsigned)(r * nb + b);
                    me.bdim.x = (unsigned)threads;
                    me.gdim.x = (unsigned)nb;
                    me.block = ctx;
                    Body::Run(w.ranks[(size_t)r].comm, args[(size_t)r], b, nb);
                });
            }
        }
    }
    for (std::thread& t : pool) t.join();
    for (hostshim::BlockCtx* c : blocks) { pthread_barrier_destroy(&c->bar); delete c; }
}

// A stream of launches: every rank runs the operators one after the other, and only ITS OWN blocks wait for one
// another between two operators (a kernel boundary on that rank's stream).  Nothing lines the ranks up, so a fast
// rank is inside operator n + 1 while a slow one still finishes operator n - what real GPUs do between two
// stream-ordered kernels, and what the forms without a closing barrier have to survive.
struct StreamOp {
    int nb;
    std::function<void(int rank, int block)> run;
};
void LaunchStream(World& w, const std::vector<StreamOp>& ops, int threads)
{
    int maxNb = 1;
    for (const StreamOp& o : ops) maxNb = std::max(maxNb, o.nb);
    std::vector<hostshim::BlockCtx*> blocks;
    std::vector<pthread_barrier_t*> boundaries;
    std::vector<std::thread> pool;
    for (int r = 0; r < w.p; ++r) {
        pthread_barrier_t* boundary = new pthread_barrier_t;
        pthread_barrier_init(boundary, nullptr, (unsigned)(maxNb * threads));
        boundaries.push_back(boundary);
        for (int b = 0; b < maxNb; ++b) {
            hostshim::BlockCtx* ctx = new hostshim::BlockCtx();
            memset(ctx->shared, 0, sizeof(ctx->shared));
            pthread_barrier_init(&ctx->bar, nullptr, (unsigned)threads);
            blocks.push_back(ctx);
            for (int t = 0; t < threads; ++t) {
                pool.emplace_back([&ops, ctx, boundary, r, b, t, threads] {
                    hostshim::ThreadCtx& me = hostshim::Tls();
                    me.tid.x = (unsigned)t;
                    me.bdim.x = (unsigned)threads;
                    me.block = ctx;
                    for (const StreamOp& o : ops) {
                        if (b < o.nb) {
                            me.bid.x = (unsigned)(r * o.nb + b);
                            me.gdim.x = (unsigned)o.nb;
                            o.run(r, b);
                        }
                        pthread_barrier_wait(boundary);
                    }
                });
            }
        }
    }
    for (std::thread& t : pool) t.join();
    for (hostshim::BlockCtx* c : blocks) { pthread_barrier_destroy(&c->bar); delete c; }
    for (pthread_barrier_t* bq : boundaries) { pthread_barrier_destroy(bq); delete bq; }
}

std::vector<float> RandVec(size_t n, unsigned seed)
{
    std::vector<float> v(n);
    unsigned s = seed * 2654435761u + 12345u;
    for (size_t i = 0; i < n; ++i) { s = s * 1664525u + 1013904223u; v[i] = (float)((s >> 8) & 0xFFFF) / 65536.0f - 0.5f; }
    return v;
}

int g_failures = 0;
void Check(bool ok, const std::string& what)
{
    if (!ok) { ++g_failures; fprintf(stderr, "FAILED: %s\n", what.c_str()); }
}
bool Close(const std::vector<float>& got, const std::vector<double>& want, double tol)
{
    for (size_t i = 0; i < want.size(); ++i)
        if (std::fabs((double)got[i] - want[i]) > tol * (1.0 + std::fabs(want[i]))) { fprintf(stderr, "  element %zu: got %g want %g\n", i, got[i], want[i]); return false; }
    return true;
}

CollArgs Zero()
{
    CollArgs a;
    memset(&a, 0, sizeof(a));
    return a;
}
void FillStage(const World& w, CollArgs& a)
{
    for (int q = 0; q < w.p; ++q) { a.src[q] = w.stageIn(q); a.xch[q] = w.xch(q); }
    a.srcMc = w.mcBase + kSlabDataOff;
}

constexpr int kNb = 2, kThreadsPerBlock = 64;

// ---------------------------------------------------------------------------------------------------------------
template <class Body>
void RunAllReduce(World& w, const char* name, size_t n, uint32_t mode, bool direct, double tol, bool nvls = false)
{
    const int p = w.p;
    for (int rep = 0; rep < 2; ++rep) {
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        std::vector<double> want(n, 0.0);
        for (int r = 0; r < p; ++r) {
            in[(size_t)r] = RandVec(n, 100u * (unsigned)rep + (unsigned)r);
            out[(size_t)r].assign(n, -1.f);
            for (size_t i = 0; i < n; ++i) want[i] += in[(size_t)r][i];
        }
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)in[(size_t)r].data();
            a.out = (char*)out[(size_t)r].data();
            a.bytes = n * sizeof(float);
            a.op = RED_SUM;
            FillStage(w, a);
            a.mode = mode;
            if (direct) {
                for (int q = 0; q < p; ++q) { a.src[q] = (const char*)in[(size_t)q].data(); a.dst[q] = (char*)out[(size_t)q].data(); }
            } else if (nvls) {
                for (int q = 0; q < p; ++q) a.dst[q] = a.xch[q];
                a.dstMc = w.mcBase + kSlabDataOff + kXchOff;
            }
            args[(size_t)r] = a;
        }
        Launch<Body>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), std::string(name) + ": a wait ran out");
        for (int r = 0; r < p; ++r) Check(Close(out[(size_t)r], want, tol), std::string(name) + " rank " + std::to_string(r) + " rep " + std::to_string(rep));
    }
}

template <class Body>
void RunReduceScatter(World& w, const char* name, size_t per, bool ll)
{
    const int p = w.p;
    for (int rep = 0; rep < 2; ++rep) {
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        std::vector<double> total(per * (size_t)p, 0.0);
        for (int r = 0; r < p; ++r) {
            in[(size_t)r] = RandVec(per * (size_t)p, 300u + 10u * (unsigned)rep + (unsigned)r);
            out[(size_t)r].assign(per, -1.f);
            for (size_t i = 0; i < total.size(); ++i) total[i] += in[(size_t)r][i];
        }
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)in[(size_t)r].data();
            a.out = (char*)out[(size_t)r].data();
            a.op = RED_SUM;
            FillStage(w, a);
            const uint64_t pair = per * sizeof(float);
            if (ll) {
                a.bytes = pair;
                for (int q = 0; q < p; ++q) { a.cnt2[q] = a.cnt[q] = pair; a.dsp2[q] = pair * (uint64_t)q; }
                a.cnt2[r] = 0;
            } else {
                a.mode = MODE_STAGE_IN;
                const uint64_t slot = (pair + 15) & ~(uint64_t)15;
                for (int q = 0; q < p; ++q) { a.cnt[q] = pair; a.dsp2[q] = pair * (uint64_t)q; a.dsp[q] = slot * (uint64_t)q; }
                a.bytes = pair * (uint64_t)p;
            }
            args[(size_t)r] = a;
        }
        Launch<Body>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), std::string(name) + ": a wait ran out");
        for (int r = 0; r < p; ++r) {
            std::vector<double> want(total.begin() + (long)(per * (size_t)r), total.begin() + (long)(per * (size_t)(r + 1)));
            Check(Close(out[(size_t)r], want, 1e-5), std::string(name) + " rank " + std::to_string(r));
        }
    }
}

template <class Body>
void RunAllGather(World& w, const char* name, size_t per, bool ll)
{
    const int p = w.p;
    for (int rep = 0; rep < 2; ++rep) {
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        for (int r = 0; r < p; ++r) { in[(size_t)r] = RandVec(per, 500u + 10u * (unsigned)rep + (unsigned)r); out[(size_t)r].assign(per * (size_t)p, -1.f); }
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)in[(size_t)r].data();
            a.out = (char*)out[(size_t)r].data();
            FillStage(w, a);
            for (int q = 0; q < p; ++q) { a.cnt[q] = per * sizeof(float); a.dsp[q] = per * sizeof(float) * (uint64_t)q; }
            a.bytes = a.cnt[r];
            if (!ll) a.mode = MODE_STAGE_IN;
            args[(size_t)r] = a;
        }
        Launch<Body>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), std::string(name) + ": a wait ran out");
        for (int r = 0; r < p; ++r)
            for (int q = 0; q < p; ++q)
                Check(memcmp(out[(size_t)r].data() + per * (size_t)q, in[(size_t)q].data(), per * sizeof(float)) == 0,
                      std::string(name) + " rank " + std::to_string(r) + " block " + std::to_string(q));
    }
}

template <class Body>
void RunBroadcast(World& w, const char* name, size_t n, uint32_t mode, int form /*0 staged pull, 1 LL, 2 nvls staged*/)
{
    const int p = w.p;
    for (int rep = 0; rep < 4; ++rep) {          // several in a row with a moving root
        const int root = rep % p;
        std::vector<std::vector<float>> buf((size_t)p);
        for (int r = 0; r < p; ++r) buf[(size_t)r] = r == root ? RandVec(n, 700u + (unsigned)rep) : std::vector<float>(n, -1.f);
        const std::vector<float> want = buf[(size_t)root];
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)buf[(size_t)r].data();
            a.out = (char*)buf[(size_t)r].data();
            a.bytes = n * sizeof(float);
            a.root = root;
            FillStage(w, a);
            if (form == 0) a.mode = MODE_STAGE_IN | mode;
            else if (form == 1) {
                if (r == root) { for (int q = 0; q < p; ++q) a.cnt2[q] = q == r ? 0 : a.bytes; }
                else a.cnt[root] = a.bytes;
            } else {
                a.dstMc = w.mcBase + kSlabDataOff + kXchOff;
            }
            args[(size_t)r] = a;
        }
        Launch<Body>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), std::string(name) + ": a wait ran out");
        for (int r = 0; r < p; ++r) Check(buf[(size_t)r] == want, std::string(name) + " rank " + std::to_string(r) + " root " + std::to_string(root));
    }
}

void RunReduceAndScatter(World& w, size_t n)
{
    const int p = w.p;
    for (uint32_t oneShot = 0; oneShot < 2; ++oneShot) {
        const int root = (int)oneShot % p;
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        std::vector<double> want(n, 0.0);
        for (int r = 0; r < p; ++r) {
            in[(size_t)r] = RandVec(n, 800u + (unsigned)r);
            out[(size_t)r].assign(n, -1.f);
            for (size_t i = 0; i < n; ++i) want[i] += in[(size_t)r][i];
        }
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)in[(size_t)r].data();
            a.out = (char*)out[(size_t)r].data();
            a.bytes = n * sizeof(float);
            a.op = RED_SUM;
            a.root = root;
            FillStage(w, a);
            a.mode = MODE_STAGE_IN | (oneShot ? MODE_PUSH : 0u);
            args[(size_t)r] = a;
        }
        Launch<ReduceBody<float>>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), "reduce: a wait ran out");
        Check(Close(out[(size_t)root], want, 1e-5), std::string("reduce ") + (oneShot ? "one-shot" : "two-shot"));
    }
    // scatter
    const int root = p - 1;
    std::vector<float> src = RandVec(n * (size_t)p, 900u);
    std::vector<std::vector<float>> out((size_t)p, std::vector<float>(n, -1.f));
    std::vector<CollArgs> args((size_t)p);
    for (int r = 0; r < p; ++r) {
        CollArgs a = Zero();
        a.in = (const char*)src.data();
        a.out = (char*)out[(size_t)r].data();
        a.bytes = n * sizeof(float);
        a.root = root;
        FillStage(w, a);
        a.mode = MODE_STAGE_IN;
        const uint64_t slot = (a.bytes + 15) & ~(uint64_t)15;
        for (int q = 0; q < p; ++q) { a.dsp2[q] = a.bytes * (uint64_t)q; a.dsp[q] = slot * (uint64_t)q; }
        args[(size_t)r] = a;
    }
    Launch<ScatterBody>(w, args, kNb, kThreadsPerBlock);
    Check(!w.failed(), "scatter: a wait ran out");
    for (int r = 0; r < p; ++r) Check(memcmp(out[(size_t)r].data(), src.data() + n * (size_t)r, n * sizeof(float)) == 0, "scatter rank " + std::to_string(r));
}

// AlltoAllV with uneven counts.  mode 0: staged in one pass; 1: read in place from the peers' buffers; 2: staged
// through windows far smaller than the pairs (several passes).
void RunAllToAllV(World& w, int mode)
{
    const int p = w.p;
    for (int rep = 0; rep < 2; ++rep) {
        auto cnt = [&](int from, int to) { return (size_t)(1000 + 37 * ((from + 2 * to + rep) % 5) + (from == 0 && to == p - 1 ? -1000 : 0)); };
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        for (int r = 0; r < p; ++r) {
            size_t s = 0, g = 0;
            for (int q = 0; q < p; ++q) { s += cnt(r, q); g += cnt(q, r); }
            in[(size_t)r] = RandVec(s, 1100u + (unsigned)r + 10u * (unsigned)rep);
            out[(size_t)r].assign(g, -1.f);
        }
        std::vector<CollArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            CollArgs a = Zero();
            a.in = (const char*)in[(size_t)r].data();
            a.out = (char*)out[(size_t)r].data();
            FillStage(w, a);
            uint64_t so = 0, ro = 0;
            for (int q = 0; q < p; ++q) {
                a.cnt2[q] = cnt(r, q) * 4; a.dsp2[q] = so; so += a.cnt2[q];
                a.cnt[q] = cnt(q, r) * 4; a.dsp[q] = ro; ro += a.cnt[q];
            }
            if (mode == 1) { for (int q = 0; q < p; ++q) a.src[q] = (const char*)in[(size_t)q].data(); }
            else a.mode = MODE_STAGE_IN;
            if (mode == 2) a.chunk = 1024;           // 256 floats per pass: five passes for the largest pair
            args[(size_t)r] = a;
        }
        Launch<A2aBody>(w, args, kNb, kThreadsPerBlock);
        Check(!w.failed(), "alltoallv: a wait ran out");
        for (int r = 0; r < p; ++r) {
            size_t ro = 0;
            for (int q = 0; q < p; ++q) {
                size_t so = 0;
                for (int t = 0; t < r; ++t) so += cnt(q, t);
                Check(memcmp(out[(size_t)r].data() + ro, in[(size_t)q].data() + so, cnt(q, r) * 4) == 0,
                      "alltoallv mode " + std::to_string(mode) + " block " + std::to_string(q) + "->" + std::to_string(r));
                ro += cnt(q, r);
            }
        }
    }
}

void RunP2pRing(World& w, size_t n)
{
    const int p = w.p;
    for (int rep = 0; rep < 2; ++rep) {
        std::vector<std::vector<float>> in((size_t)p), out((size_t)p);
        for (int r = 0; r < p; ++r) { in[(size_t)r] = RandVec(n, 1300u + (unsigned)r); out[(size_t)r].assign(n, -1.f); }
        std::vector<P2pArgs> args((size_t)p);
        for (int r = 0; r < p; ++r) {
            P2pArgs a;
            memset(&a, 0, sizeof(a));
            a.nItems = 2;
            a.items[0] = P2pItem{(char*)in[(size_t)r].data(), n * 4, (r + 1) % p, 1};
            a.items[1] = P2pItem{(char*)out[(size_t)r].data(), n * 4, (r + p - 1) % p, 0};
            a.halfBytes = kMailboxHalf;
            a.mailboxOff = kMailboxOff;
            a.seq = w.ranks[(size_t)r].p2pSeq;
            args[(size_t)r] = a;
        }
        Launch<P2pBody>(w, args, 2, kThreadsPerBlock);
        Check(!w.failed(), "send/recv: a wait ran out");
        for (int r = 0; r < p; ++r) Check(out[(size_t)r] == in[(size_t)((r + p - 1) % p)], "send/recv ring rank " + std::to_string(r));
    }
}

#include "harness_ext.inc"

void RunWorld(int p, bool quick)
{
    printf("== %d ranks\n", p);
    fflush(stdout);
    World w(p);
    const size_t n = quick ? 3001 : 20011;
    RunAllReduce<ArTwoShotBody<float>>(w, "allreduce two-shot staged", n, MODE_STAGE_IN, false, 1e-5);
    RunAllReduce<ArTwoShotBody<float>>(w, "allreduce two-shot in place on the peers, pushed out", n, MODE_PUSH, true, 1e-5);
    RunAllReduce<ArOneShotBody<float>>(w, "allreduce one-shot staged", n, MODE_STAGE_IN, false, 1e-5);
    RunAllReduce<ArLLBody<float>>(w, "allreduce flag-in-data", 1501, 0, false, 1e-5);
    RunAllReduce<ArNvlsBody<float>>(w, "allreduce switch", (n + 3) / 4 * 4, MODE_STAGE_IN | MODE_STAGE_OUT, false, 1e-5, true);
    RunReduceScatter<RsBody<float>>(w, "reducescatter", n / 4, false);
    RunReduceScatter<RsNvlsBody<float>>(w, "reducescatter switch", (n / 4 + 3) / 4 * 4, false);
    RunReduceScatter<LLExchangeBody<float, true>>(w, "reducescatter flag-in-data", 701, true);
    RunAllGather<AgBody>(w, "allgather", n / 4, false);
    RunAllGather<AgLLBody>(w, "allgather flag-in-data", 701, true);
    RunBroadcast<BcastBody>(w, "broadcast two-shot", n, 0, 0);
    RunBroadcast<BcastBody>(w, "broadcast one-shot", n, MODE_PUSH, 0);
    RunBroadcast<LLExchangeBody<int8_t, false>>(w, "broadcast flag-in-data", 1201, 0, 1);
    RunBroadcast<BcastNvlsBody>(w, "broadcast switch", n, 0, 2);
    RunReduceAndScatter(w, n / 2);
    for (int mode = 0; mode < 3; ++mode) RunAllToAllV(w, mode);
    RunP2pRing(w, 30000);
    RunExtended(w, n);
    // mixed flag-in-data operators in a row: broadcast, allreduce, broadcast from another root ...
    for (int it = 0; it < 3; ++it) {
        RunBroadcast<LLExchangeBody<int8_t, false>>(w, "mixed: broadcast flag-in-data", 257, 0, 1);
        RunAllReduce<ArLLBody<float>>(w, "mixed: allreduce flag-in-data", 129, 0, false, 1e-5);
    }
}

// Small sizes around the vector, line and slice boundaries (1 ... 257 elements) for the bodies whose slicing rounds to 16
// bytes: the last slices are short or empty, block rows get nothing, tails are shorter than a vector.  Meant for the
// AddressSanitizer build (bounds), quick enough for ThreadSanitizer too.
void RunEdges(int p, bool all)
{
    printf("== edges, %d ranks\n", p);
    fflush(stdout);
    World w(p);
    const std::vector<size_t> every = {1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 33, 63, 65, 127, 129, 255, 257}, few = {1, 3, 8, 17, 65, 257};
    for (size_t n : all ? every : few) {
        RunAllReduce<ArTwoShotBody<float>>(w, "edges: allreduce two-shot staged", n, MODE_STAGE_IN, false, 1e-5);
        RunAllReduce<ArOneShotBody<float>>(w, "edges: allreduce one-shot staged", n, MODE_STAGE_IN, false, 1e-5);
        RunAllReduce<ArLLBody<float>>(w, "edges: allreduce flag-in-data", n, 0, false, 1e-5);
        RunReduceScatter<RsBody<float>>(w, "edges: reducescatter", n, false);
        RunAllGather<AgBody>(w, "edges: allgather", n, false);
        RunBroadcast<BcastBody>(w, "edges: broadcast two-shot", n, 0, 0);
        RunBroadcast<BcastBody>(w, "edges: broadcast one-shot", n, MODE_PUSH, 0);
        RunPushReduceScatter(w, n, 0);
        RunPushReduceScatter(w, n, 1);
        RunPushAllReduce(w, n, false);
        RunAllToAllPush(w, n);
        RunBroadcastPipe(w, n, false, 2);
        RunBroadcastPipe(w, n, true, 3);
    }
}

}  // namespace

int main(int argc, char** argv)
{
    const bool quick = argc > 1 && std::string(argv[1]) == "--quick";
    if (argc > 1 && (std::string(argv[1]) == "--edges" || std::string(argv[1]) == "--edges-all")) {
        const bool all = std::string(argv[1]) == "--edges-all";          // every size on 2, 3 and 5 ranks: several minutes
        for (int p : {2, 3, 5}) {
            if (p == 5 && !all) continue;
            RunEdges(p, all);
        }
        if (g_failures) { fprintf(stderr, "%d check(s) failed\n", g_failures); return 1; }
        printf("kernel harness: all checks passed\n");
        return 0;
    }
    for (int p : {2, 3, 8}) RunWorld(p, quick || p == 8);
    if (g_failures) { fprintf(stderr, "%d check(s) failed\n", g_failures); return 1; }
    printf("kernel harness: all checks passed\n");
    return 0;
}
