// Host engine internals: the world of simulated ranks, the primitive layer the
// algorithm templates are written against, and the recorded trace.
//
// Primitive layer = the role of the reference's alg_data_trans_wrapper
// (Send/Recv x Write/Read x Reduce, LocalCopy, LocalReduce, notify record /
// wait, alg_data_trans_wrapper.h:23-84).  A template names memory by
// (rank, buffer kind, offset): INPUT and OUTPUT are the user buffers of the
// current operator, SCRATCH is the rank's staging buffer (the CCL buffer).
// The trace mirrors the analyzer's TaskStub list (sim_world/sim_task.h:22-24):
// LOCAL_COPY, LOCAL_REDUCE, READ, READ_REDUCE, WRITE, WRITE_REDUCE, POST, WAIT.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>
#include "../algo/step_tables.h"
#include "../topo/topo.h"
#include "hccl/hccl_types.h"

namespace hccl {

class CommImpl;
struct OpParam;

enum class BufKind : uint8_t { INPUT = 0, OUTPUT = 1, SCRATCH = 2 };
struct Mem {
    uint32_t rank;
    BufKind buf;
    uint64_t off;     // bytes
};
inline Mem In(uint32_t r, uint64_t off = 0) { return {r, BufKind::INPUT, off}; }
inline Mem Out(uint32_t r, uint64_t off = 0) { return {r, BufKind::OUTPUT, off}; }
inline Mem Scratch(uint32_t r, uint64_t off = 0) { return {r, BufKind::SCRATCH, off}; }

enum class TaskKind : uint8_t { LOCAL_COPY, LOCAL_REDUCE, READ, READ_REDUCE, WRITE, WRITE_REDUCE, POST, WAIT };
struct Task {
    TaskKind kind;
    uint32_t rank;       // executing rank
    uint32_t queue;      // execution queue of that rank (tasks of one queue are ordered)
    Mem dst, src;        // data tasks
    uint64_t bytes;
    uint32_t peer;       // POST / WAIT
    uint32_t notifyIdx;
};

struct HostOpDesc {
    HcclCMDType op;
    HcclDataType dtype;
    HcclReduceOp redOp;
    uint64_t count;                    // elements (meaning per op, as in the C API)
    uint32_t root;
    std::vector<uint64_t> sendCounts, sdispls, recvCounts, rdispls;   // elements
};

class HostWorld;

// What a template sees.  One instance per rank and operator call.
class HostPrims {
public:
    HostPrims(HostWorld* w, uint32_t rank) : w_(w), me_(rank) {}
    uint32_t me() const { return me_; }
    // dst / src may live on any rank; at least one side must be this rank.
    void Copy(Mem dst, Mem src, uint64_t bytes, uint32_t queue = 0);
    void Reduce(Mem dst, Mem src, uint64_t bytes, uint32_t queue = 0);   // dst = dst (op) src
    void Post(uint32_t peer, uint32_t idx, uint32_t queue = 0);
    void Wait(uint32_t peer, uint32_t idx, uint32_t queue = 0);
    // Barrier-like handshakes built from Post / Wait over a group of ranks.
    void SyncGroup(const std::vector<uint32_t>& group, uint32_t idx, uint32_t queue = 0);
    bool failed() const { return failed_; }
private:
    void Record(const Task& t);
    HostWorld* w_;
    uint32_t me_;
    bool failed_ = false;
};

struct VerifyReport {
    bool ok = true;
    uint64_t tasks = 0, edges = 0, dataTasks = 0;
    std::vector<std::string> errors;
    std::string Text() const;
};

class HostWorld {
public:
    HostWorld(uint32_t nRanks, const TopoMeta& meta, uint64_t scratchBytes, uint64_t timeoutNs);
    ~HostWorld();
    uint32_t nRanks() const { return n_; }
    const TopoInfo& Topo(uint32_t rank) const { return topo_[rank]; }
    uint64_t scratchBytes() const { return scratchBytes_; }

    // Entry of an operator on one rank: publishes the rank's buffers, waits for all ranks, checks that every rank
    // called the same operator with compatible parameters, then lets the caller run its template.
    HcclResult Enter(uint32_t rank, const HostOpDesc& d, const void* in, void* out, uint64_t inBytes, uint64_t outBytes);
    HcclResult Leave(uint32_t rank);
    HcclResult BarrierAll(uint32_t rank);     // host-side rendezvous with timeout (a rank that never arrives -> TIMEOUT)
    void Abort(const std::string& why);
    bool aborted() const { return aborted_.load(); }
    // Recovery point of the operator retry: every rank calls it after a failed attempt.  When the last rank arrives
    // the abort state, the notify counters and the rendezvous are cleared so that the operator can be issued again
    // from its inputs.  A rank that never arrives -> HCCL_E_TIMEOUT on the others (the retry has failed).
    HcclResult Recover(uint32_t rank);
    // Test hook: the next `count` notifies posted by `rank` are lost on the way (a dropped message).
    void DropPosts(uint32_t rank, uint32_t count) { dropPosts_[rank].store(count); }
    uint64_t recoveries() const { return recoverGen_; }

    char* Resolve(const Mem& m) const;
    uint64_t BufBytes(uint32_t rank, BufKind k) const;
    const HostOpDesc& CurrentOp() const { return cur_; }

    // notifies
    void Post(uint32_t from, uint32_t to, uint32_t idx);
    bool Wait(uint32_t me, uint32_t from, uint32_t idx);

    // trace
    void TraceBegin();
    bool tracing() const { return tracing_.load(); }
    void Append(const Task& t);
    VerifyReport Verify();      // checks the trace of the operators run since TraceBegin, then stops tracing
    // Checks a hand-written trace of one operator (self-tests of the verifier): tasks[r] is rank r's task list.
    VerifyReport VerifyTasks(const HostOpDesc& d, uint64_t inBytes, uint64_t outBytes, const std::vector<std::vector<Task>>& tasks);

    void AddRef() { refs_.fetch_add(1); }
    bool Release() { return refs_.fetch_sub(1) == 1; }
    static constexpr uint32_t kNotifyIdx = 8;

private:
    struct OpRecord {
        HostOpDesc desc;
        std::vector<uint64_t> inBytes, outBytes;
        std::vector<std::vector<Task>> tasks;     // per rank
    };
    uint32_t n_;
    std::vector<TopoInfo> topo_;
    uint64_t scratchBytes_, timeoutNs_;
    std::vector<std::unique_ptr<char[]>> scratch_;
    std::vector<const void*> in_;
    std::vector<void*> out_;
    std::vector<uint64_t> inBytes_, outBytes_;
    std::vector<HostOpDesc> descs_;
    HostOpDesc cur_;
    // rendezvous
    std::mutex mu_;
    std::condition_variable cv_;
    uint32_t arrived_ = 0;
    uint64_t generation_ = 0;
    uint32_t recoverArrived_ = 0;
    uint64_t recoverGen_ = 0;
    std::vector<std::atomic<uint32_t>> dropPosts_;
    std::atomic<bool> aborted_{false};
    std::string abortWhy_;
    // notify counters: [to][from][idx] posted, and per-waiter consumed counts
    std::vector<std::atomic<uint64_t>> posted_;
    std::vector<uint64_t> consumed_;
    // trace
    std::atomic<bool> tracing_{false};
    std::mutex traceMu_;
    std::vector<OpRecord> ops_;
    std::atomic<int> refs_{0};
    friend class HostVerifier;
};

class HostRank {
public:
    HostRank(std::shared_ptr<HostWorld> w, uint32_t rank) : world(std::move(w)), rank(rank) {}
    std::shared_ptr<HostWorld> world;
    uint32_t rank;
};

// Algorithm identifiers of the host engine (what AlgEntry::hostAlg holds).
enum HostAlg : int {
    HALG_AR_MESH_ONESHOT = 0, HALG_AR_MESH_TWOSHOT, HALG_AR_RING, HALG_AR_RHD, HALG_AR_NHR, HALG_AR_SEQ_MESH_RING, HALG_AR_SEQ_MESH_NHR,
    HALG_AR_SEQ_MESH_RHD, HALG_AR_SEQ3_MESH_NHR_NHR, HALG_AR_SEQ_SQUEEZE2D_MESH_MESH, HALG_AR_PARALLEL_MESH_NHR, HALG_AR_ORDER_PRESERVED,
    HALG_RS_MESH, HALG_RS_RING, HALG_RS_RHD, HALG_RS_NHR, HALG_RS_SEQ_MESH_NHR, HALG_RS_ORDER_PRESERVED,
    HALG_AG_MESH, HALG_AG_RING, HALG_AG_RHD, HALG_AG_NHR, HALG_AG_SEQ_MESH_NHR,
    HALG_BCAST_MESH_ONESHOT, HALG_BCAST_MESH_TWOSHOT, HALG_BCAST_NHR,
    HALG_REDUCE_MESH_ONESHOT, HALG_REDUCE_MESH_TWOSHOT, HALG_REDUCE_NHR,
    HALG_SCATTER_MESH, HALG_SCATTER_NHR, HALG_SCATTER_RING,
    HALG_A2A_MESH, HALG_A2A_PAIRWISE,
    HALG_P2P_DIRECT, HALG_BARRIER_MESH, HALG_BARRIER_NHR, HALG_BARRIER_RHD,
    // executors of host_executors.cc
    HALG_AR_CONCURRENT_MESH_NHR, HALG_RS_CONCURRENT_MESH_NHR, HALG_AG_CONCURRENT_MESH_NHR,
    HALG_AG_MESH_DETOUR, HALG_RS_MESH_DETOUR, HALG_SCATTER_MESH_DETOUR,
    HALG_AR_PIPELINE_MESH_NHR, HALG_AR_PIPELINE3_MESH_NHR_NHR, HALG_AG_PIPELINE_MESH_MESH, HALG_RS_PIPELINE_MESH_MESH, HALG_BCAST_PIPELINE_MESH_MESH,
    HALG_AG_NB, HALG_BCAST_NB, HALG_SCATTER_NB,
    HALG_A2A_HIER,
    HALG_BCAST_SEQ_MESH_NHR, HALG_REDUCE_SEQ_MESH_NHR, HALG_SCATTER_SEQ_MESH_MESH, HALG_BARRIER_SEQ_MESH_NHR,
    HALG_AR_TREE,
    HALG_BCAST_RING, HALG_BCAST_RHD, HALG_REDUCE_RING, HALG_REDUCE_RHD,
    HALG_RS_SEQ_MESH_RING, HALG_RS_SEQ_MESH_RHD, HALG_AG_SEQ_MESH_RING, HALG_AG_SEQ_MESH_RHD,
    HALG_A2A_SERIAL, HALG_REDUCE_PIPELINE_MESH_NHR, HALG_SCATTER_PIPELINE_MESH_MESH,
    HALG_AG_PARALLEL_MESH_MESH, HALG_RS_PARALLEL_MESH_MESH, HALG_BCAST_CONCURRENT_MESH_NHR, HALG_REDUCE_CONCURRENT_MESH_NHR,
    HALG_AR_SEQ_2DIE_MESH_MESH, HALG_AR_SOLE_MESH_CONCUR,
    HALG_BCAST_PARALLEL_MESH_MESH, HALG_SCATTER_PARALLEL_MESH_MESH, HALG_REDUCE_PARALLEL_MESH_NHR, HALG_A2A_CONCURRENT_MESH_MESH,
    HALG_AG_PIPELINE3_MESH_MESH_MESH, HALG_RS_PIPELINE3_MESH_MESH_MESH, HALG_AG_SEQ3_MESH_NHR_NHR, HALG_RS_SEQ3_MESH_NHR_NHR, HALG_SCATTER_CONCURRENT_MESH_MESH,
    HALG_COUNT
};
// Runs host algorithm `alg` for this rank; the world is already inside Enter().
HcclResult RunHostAlgorithm(HostWorld& w, uint32_t rank, int alg, const OpParam& p);
// Scratch bytes the algorithm needs for this call (0 = none); the sole executor loops when a call exceeds the buffer.
uint64_t HostScratchMultiple(int alg, uint32_t nRanks);

}  // namespace hccl
