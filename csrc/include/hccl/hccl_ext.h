// Extensions of hccl_b200 beyond the HCCL API surface: host-simulated
// communicators, introspection of the selector, profiling records and test
// hooks.  Everything here is optional for a user who only ports HCCL code.
#ifndef HCCL_B200_EXT_H_
#define HCCL_B200_EXT_H_

#include "hccl_types.h"

#ifdef __cplusplus
extern "C" {
#endif

// `nRanks` host-engine communicators in this process (ranks = caller threads,
// buffers = host memory).  topoJson: "[[[0,1,2,3],[4,5,6,7]]]" (pods > servers >
// devices) or NULL for one server.  Each rank's calls must come from its own
// thread, as with one process per rank.
HcclResult HcclCommInitHostSim(uint32_t nRanks, const char* topoJson, const HcclCommConfig* config, HcclComm* comms);
// Emulated device communicators: `nRanks` ranks on the CURRENT GPU; every
// collective runs as one cooperative kernel once all ranks have called it (call
// the ranks one after the other from one thread).
HcclResult HcclCommInitEmulated(uint32_t nRanks, const HcclCommConfig* config, HcclComm* comms);

// Name of the algorithm the last operator on this communicator ran with.
/* Reductions fused with a data type cast and a scale: out[i] = (outType)(scale * reduce_r in_r[i]), accumulated in fp32.
 * inType and outType are each one of fp32, bf16, fp16.  Typical uses: averaging gradients (scale = 1 / ranks) without
 * a second pass, reducing bf16 gradients into an fp32 master copy, reducing fp32 partials into a bf16 tensor.  The
 * nearest analogue in the reference widens hif8 to float, reduces and narrows again inside one ReduceScatter kernel
 * (aiv_reduce_scatter_mesh_1d_hif8.h).  The output needs count (AllReduce) or recvCount (ReduceScatter) elements of
 * outType; an output that overlaps the input is only allowed when the types have the same size. */
HcclResult HcclAllReduceEx(void* sendBuf, void* recvBuf, uint64_t count, HcclDataType inType, HcclDataType outType, HcclReduceOp op, float scale,
                           HcclComm comm, hcclStream_t stream);
HcclResult HcclReduceScatterEx(void* sendBuf, void* recvBuf, uint64_t recvCount, HcclDataType inType, HcclDataType outType, HcclReduceOp op,
                               float scale, HcclComm comm, hcclStream_t stream);

HcclResult HcclGetLastAlgName(HcclComm comm, char* name, uint32_t capacity);
// Runs selection for a hypothetical call and writes the cost table as text.
HcclResult HcclSelectorExplain(HcclComm comm, HcclCMDType op, uint64_t count, HcclDataType dataType,
                               HcclReduceOp reduceOp, int registered, char* text, uint32_t capacity);
// Number of registered algorithms; and name / op / engine of entry i.
uint32_t HcclAlgRegistryCount(void);
HcclResult HcclAlgRegistryEntry(uint32_t index, char* name, uint32_t capacity, HcclCMDType* op, HcclCommEngine* engine);

// Profiling ring (HCCL_PROFILING=1 host timing, =2 plus device time).
HcclResult HcclProfilingSetLevel(int level);
HcclResult HcclProfilingDump(char* text, uint32_t capacity);   // one line per record, CSV

// Trace + verifier of host-engine communicators: start recording on all ranks of
// the world `comm` belongs to, run operators, then verify (deadlock, bounds,
// races, semantics).  `report` receives a human-readable summary.
HcclResult HcclHostTraceBegin(HcclComm comm);
HcclResult HcclHostTraceVerify(HcclComm comm, char* report, uint32_t capacity);

// Test hook: launches a kernel that waits on a flag nothing sets; the wait must
// run out after the communicator's wait budget and surface as HCCL_E_TIMEOUT
// from HcclCommGetAsyncError.  Never traps and never spins past the budget.
HcclResult HcclTestLaunchUnsignalledWait(HcclComm comm, hcclStream_t stream);
// Test hook: the next bootstrap exchange on this rank fails as if its connection dropped.
HcclResult HcclTestInjectBootstrapFailure(HcclComm comm);
// Host-engine communicators only: the next `count` notifies this rank posts are lost (a dropped message), which makes
// the waiting peers time out; and how many times the world went through the operator-retry recovery point.
HcclResult HcclTestHostDropPosts(HcclComm comm, uint32_t count);
HcclResult HcclTestHostRecoveries(HcclComm comm, uint64_t* count);
// Plan-cache statistics.
HcclResult HcclGetPlanCacheStats(HcclComm comm, uint64_t* hits, uint64_t* misses, uint64_t* entries);
// Overrides entries of the link model the cost model uses (GB/s and microseconds); negative = keep.
HcclResult HcclSetLinkModel(double p2pGBs, double nvlsGBs, double localCopyGBs, double launchUs, double barrierUs,
                            double llHopUs);
// Resource query for graph builders (the role of HCCL's HcclCalcOpRes*GraphMode, calc_resource_graph_mode.cc:51-633:
// scratch size, stream count, task count, core count per op before it runs): which algorithm a call would use, how
// many thread blocks it launches, how many bytes of the communicator's staging slab it touches per loop and how many
// loops (kernel launches) the sole executor needs.  Ops of this library never use extra streams.
typedef struct {
    char algName[128];
    uint32_t engine;        // HcclCommEngine
    uint32_t blocks;        // thread blocks per launch
    uint32_t launches;      // kernel launches for this call (loops over the staging slab)
    uint32_t streams;       // always 1: the caller's stream
    uint64_t scratchBytes;  // bytes of the staging slab used per launch (0 with symmetric buffers)
} HcclOpResource;
HcclResult HcclCalcOpResource(HcclComm comm, HcclCMDType op, uint64_t count, HcclDataType dataType, HcclReduceOp reduceOp, int registered,
                              HcclOpResource* res);

// Selection on a synthetic one-box NVSwitch topology, no device needed (regression tests of the device cost model):
// the text of HcclSelectorExplain for `bytes` (as the selector counts them) on nRanks GPUs.  deterministic: 0, 1, 2 = strict.
HcclResult HcclDebugExplainDevice(uint32_t nRanks, int nvls, HcclCMDType op, uint64_t bytes, HcclDataType dataType, HcclReduceOp reduceOp,
                                  int registered, int deterministic, char* text, uint32_t capacity);

// The out-of-band bootstrap on its own, without a device (tests of the rendezvous and of its failure paths): connect
// `rank` of `nRanks` to the endpoint in `info` (HcclGetRootInfo), then all-gather / barrier / agree (logical AND) over
// the handle.  A rank that never connects makes the others' Connect return HCCL_E_TIMEOUT after timeoutS seconds; a
// rank that closes makes the others' next call return HCCL_E_REMOTE.
HcclResult HcclDebugBootstrapConnect(const HcclRootInfo* info, uint32_t rank, uint32_t nRanks, uint32_t timeoutS, void** handle);
HcclResult HcclDebugBootstrapAllGather(void* handle, const void* send, void* recv, uint64_t bytesPerRank);
HcclResult HcclDebugBootstrapBarrier(void* handle);
HcclResult HcclDebugBootstrapAgree(void* handle, int ok, int* all);
HcclResult HcclDebugBootstrapInjectFailure(void* handle);
HcclResult HcclDebugBootstrapClose(void* handle);

// Self-test entry of the topology model: what the literal `topoJson` ([[[devices of a server], ...] per pod]; NULL =
// one server) gives `rank`, the groups of a one / two / three level match (matchKind 0 / 1 / 2), and whether the
// serialised model survives a round trip while a damaged or truncated blob is refused.
HcclResult HcclDebugTopo(const char* topoJson, uint32_t nRanks, uint32_t rank, int matchKind, char* text, uint32_t capacity);

// Self-test entry of the trace verifier: checks a trace written as text (grammar beside the definition in
// csrc/cpu/host_comm.cc) and writes the verifier's report ("OK: ..." or "FAILED: ..." with one line per finding).
HcclResult HcclDebugVerifyTrace(const char* script, char* report, uint32_t capacity);

// Post-mortem record of the last operator entries of this process (kept when HCCL_DIAGNOSE_ENABLE=1, 2000 lines, oldest
// first), the counterpart of HCCL's diagnose ring.  Writes at most `capacity` bytes including the terminator.
HcclResult HcclDiagnoseDump(char* text, uint32_t capacity);

// Unit-test access to pure functions.  Each writes a text rendering into `text`.
//   kind "nhr_rs" / "nhr_ag" / "rhd_rs" / "rhd_ag" / "ring_rs" / "ring_ag" / "pairwise" / "fold": step table of `rank` among `p`
//   kind "parse_algo": parses `arg` as an HCCL_ALGO value;  kind "rhd_info": pairing of `rank`
HcclResult HcclDebugStepTable(const char* kind, uint32_t p, uint32_t rank, const char* arg, char* text, uint32_t capacity);
// Parses the environment-style settings given as "NAME=value\nNAME=value" and renders the resulting configuration
// (and the list of rejected variables) as text, without touching the process environment.
HcclResult HcclDebugParseEnv(const char* settings, char* text, uint32_t capacity);
// Evaluates the cost formula for one segment: (A / util(net, bytes * ratio) + B) * bytes + C, floored by D.
/* Loads link parameters and per-GPU-count utilisation curves from a measurement file (see docs/algorithms.md); the
 * library loads hccl_b200/data/link_model.json, or the file HCCL_LINK_MODEL_FILE names, by itself on first use. */
HcclResult HcclLoadLinkModel(const char* path, char* error, uint32_t capacity);
double HcclDebugLinkUtilisation(int netType, double bytes, uint32_t nRanks);
double HcclDebugEvalCost(double A, double B, double C, double D, int netType, double ratio, double bytes);
// Re-reads the HCCL_* environment variables (they are parsed once per process otherwise).  Existing communicators
// keep the plans they already cached.
HcclResult HcclReloadEnvConfig(void);
const char* HcclGetVersion(void);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_EXT_H_
