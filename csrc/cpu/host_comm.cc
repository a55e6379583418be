// placeholder until the host engine lands
#include "host_comm.h"
#include "../core/log.h"
namespace hccl {
void RegisterHostAlgorithms() {}
HcclResult HostWorldCreate(uint32_t, const char*, const HcclCommConfig*, CommImpl**) { return HCCL_E_NOT_SUPPORT; }
void HostRankRelease(HostRank*) {}
HcclResult HostExecOp(CommImpl*, OpParam&) { return HCCL_E_NOT_SUPPORT; }
}
#include "hccl/hccl_ext.h"
extern "C" {
HcclResult HcclHostTraceBegin(HcclComm) { return HCCL_E_NOT_SUPPORT; }
HcclResult HcclHostTraceVerify(HcclComm, char*, uint32_t) { return HCCL_E_NOT_SUPPORT; }
}
