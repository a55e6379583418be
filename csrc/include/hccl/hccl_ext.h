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
// Plan-cache statistics.
HcclResult HcclGetPlanCacheStats(HcclComm comm, uint64_t* hits, uint64_t* misses, uint64_t* entries);
// Overrides entries of the link model the cost model uses (GB/s and microseconds); negative = keep.
HcclResult HcclSetLinkModel(double p2pGBs, double nvlsGBs, double localCopyGBs, double launchUs, double barrierUs,
                            double llHopUs);
// Re-reads the HCCL_* environment variables (they are parsed once per process otherwise).  Existing communicators
// keep the plans they already cached.
HcclResult HcclReloadEnvConfig(void);
const char* HcclGetVersion(void);

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_EXT_H_
