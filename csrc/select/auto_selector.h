// Threshold-tree selection: one hand-written decision tree per operator.
//
// The reference keeps such trees beside its cost-model selector
// (execute_selector.{cc,h}, auto_selector_base.{cc,h}, one
// src/ops/<op>/selector/*_auto_selector.cc per operator) and uses them where
// the cost model has no calibration - level-0 topologies that are not a 1-D
// mesh, and operators issued on behalf of fused matmul kernels
// (op_common.cc:225-230).  Its trees cut on message size (AllReduce: one-shot
// up to 16 KiB, "small" up to 512 KiB, "large" from 1 MiB,
// all_reduce_auto_selector.cc:32-57, auto_selector_base.h:23-26), on the rank
// count (power of two -> halving-doubling, else NHR) and on the number of
// topology levels.
//
// Here the tree is used when HCCL_SELECTOR_MODE=threshold, and for calls that
// come from the fused matmul kernels.  The cut points for the device engines
// are where the measured curves of the 8-GPU sweep cross; the host-engine cut
// points are the reference's.  The tree only NAMES an algorithm: the registry's
// filters still decide whether it can run, and the cost model takes over when
// it cannot.
#pragma once
#include <string>
#include "selector.h"

namespace hccl {

struct ThresholdInput {
    HcclCMDType op = HCCL_CMD_INVALID;
    uint64_t bytes = 0;           // as OpDesc::bytes
    uint32_t nRanks = 1;
    uint32_t levels = 1;          // topology levels (1 = one server)
    bool hostEngine = false;
    bool nvls = false;            // switch reduction / multicast available and the buffers have a multicast alias
    bool strictOrder = false;     // HCCL_DETERMINISTIC=strict
};

// Name of the algorithm the tree picks, empty when the tree has no opinion for this operator.
std::string ThresholdSelect(const ThresholdInput& in);
ThresholdInput ThresholdInputOf(const TopoInfo& topo, const OpDesc& op);

}  // namespace hccl
