// Argument validation shared by all operator entry points.
//
// Rule set taken from the reference: counts are bounded by SYS_MAX_COUNT
// 0x7FFFFFFFF (hccl_common.h:43; checks op_common.cc:4311-4320); value 13 and
// RESERVED are not data types (hccl_common.h:60-75); reductions reject uint8 /
// uint16 / uint32 / int128 / hif8 and the 8-bit floats except that
// ReduceScatter accepts fp8 here where the reference accepts hif8
// (op_common.cc:4330-4335); PROD only for int8, int32, int64, uint64, fp16,
// fp32, fp64 (:4394-4396); group names are at most 127 characters
// (param_check.cc:18-68).
#pragma once
#include <cstdint>
#include <string>
#include "hccl/hccl_types.h"

namespace hccl {

constexpr uint64_t kSysMaxCount = 0x7FFFFFFFFull;
constexpr uint32_t kGroupNameMaxLen = 127;

uint32_t DataTypeSize(HcclDataType t);          // 0 for invalid
bool IsValidDataType(HcclDataType t);
const char* DataTypeName(HcclDataType t);
const char* ReduceOpName(HcclReduceOp op);
const char* CmdName(HcclCMDType op);

HcclResult CheckCount(const char* opName, uint64_t count);
HcclResult CheckDataType(const char* opName, HcclDataType t, bool needReduce, bool isReduceScatter);
HcclResult CheckReduceOp(const char* opName, HcclDataType t, HcclReduceOp op);
HcclResult CheckRank(const char* opName, const char* what, uint32_t rank, uint32_t rankSize);
HcclResult CheckGroupName(const std::string& name);
HcclResult CheckTag(const std::string& tag);

}  // namespace hccl
