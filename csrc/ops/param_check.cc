#include "param_check.h"
#include "../core/log.h"

namespace hccl {

uint32_t DataTypeSize(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_HIF8: case HCCL_DATA_TYPE_FP8E4M3:
        case HCCL_DATA_TYPE_FP8E5M2: case HCCL_DATA_TYPE_FP8E8M0: return 1;
        case HCCL_DATA_TYPE_INT16: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_BFP16: return 2;
        case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_FP32: return 4;
        case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64: case HCCL_DATA_TYPE_FP64: return 8;
        case HCCL_DATA_TYPE_INT128: return 16;
        default: return 0;
    }
}
bool IsValidDataType(HcclDataType t) { return DataTypeSize(t) != 0; }

const char* DataTypeName(HcclDataType t)
{
    switch (t) {
        case HCCL_DATA_TYPE_INT8: return "int8"; case HCCL_DATA_TYPE_INT16: return "int16"; case HCCL_DATA_TYPE_INT32: return "int32";
        case HCCL_DATA_TYPE_FP16: return "float16"; case HCCL_DATA_TYPE_FP32: return "float32"; case HCCL_DATA_TYPE_INT64: return "int64";
        case HCCL_DATA_TYPE_UINT64: return "uint64"; case HCCL_DATA_TYPE_UINT8: return "uint8"; case HCCL_DATA_TYPE_UINT16: return "uint16";
        case HCCL_DATA_TYPE_UINT32: return "uint32"; case HCCL_DATA_TYPE_FP64: return "float64"; case HCCL_DATA_TYPE_BFP16: return "bfloat16";
        case HCCL_DATA_TYPE_INT128: return "int128"; case HCCL_DATA_TYPE_HIF8: return "hif8"; case HCCL_DATA_TYPE_FP8E4M3: return "fp8e4m3";
        case HCCL_DATA_TYPE_FP8E5M2: return "fp8e5m2"; case HCCL_DATA_TYPE_FP8E8M0: return "fp8e8m0";
        default: return "invalid";
    }
}
const char* ReduceOpName(HcclReduceOp op)
{
    switch (op) { case HCCL_REDUCE_SUM: return "sum"; case HCCL_REDUCE_PROD: return "prod"; case HCCL_REDUCE_MAX: return "max"; case HCCL_REDUCE_MIN: return "min"; default: return "invalid"; }
}
const char* CmdName(HcclCMDType op)
{
    switch (op) {
        case HCCL_CMD_BROADCAST: return "Broadcast"; case HCCL_CMD_ALLREDUCE: return "AllReduce"; case HCCL_CMD_REDUCE: return "Reduce";
        case HCCL_CMD_SEND: return "Send"; case HCCL_CMD_RECEIVE: return "Recv"; case HCCL_CMD_ALLGATHER: return "AllGather";
        case HCCL_CMD_REDUCE_SCATTER: return "ReduceScatter"; case HCCL_CMD_ALLTOALLV: return "AlltoAllV"; case HCCL_CMD_ALLTOALLVC: return "AlltoAllVC";
        case HCCL_CMD_ALLTOALL: return "AlltoAll"; case HCCL_CMD_SCATTER: return "Scatter"; case HCCL_CMD_BATCH_SEND_RECV: return "BatchSendRecv";
        case HCCL_CMD_ALLGATHER_V: return "AllGatherV"; case HCCL_CMD_REDUCE_SCATTER_V: return "ReduceScatterV"; case HCCL_CMD_BARRIER: return "Barrier";
        default: return "Invalid";
    }
}

HcclResult CheckCount(const char* opName, uint64_t count)
{
    if (count > kSysMaxCount) {
        ReportInputError("EI0003", opName, "count", std::to_string(count), "at most 0x7FFFFFFFF elements");
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult CheckDataType(const char* opName, HcclDataType t, bool needReduce, bool isReduceScatter)
{
    if (!IsValidDataType(t)) {
        ReportInputError("EI0003", opName, "dataType", std::to_string((int)t), "a value of HcclDataType (13 and 255 are not data types)");
        return HCCL_E_PARA;
    }
    if (!needReduce) return HCCL_SUCCESS;
    switch (t) {
        case HCCL_DATA_TYPE_UINT8: case HCCL_DATA_TYPE_UINT16: case HCCL_DATA_TYPE_UINT32: case HCCL_DATA_TYPE_INT128:
        case HCCL_DATA_TYPE_HIF8: case HCCL_DATA_TYPE_FP8E8M0:
            ReportInputError("EI0003", opName, "dataType", DataTypeName(t), "a type that supports reduction");
            return HCCL_E_NOT_SUPPORT;
        case HCCL_DATA_TYPE_FP8E4M3: case HCCL_DATA_TYPE_FP8E5M2:
            if (isReduceScatter) return HCCL_SUCCESS;
            ReportInputError("EI0003", opName, "dataType", DataTypeName(t), "8-bit floats reduce only in ReduceScatter");
            return HCCL_E_NOT_SUPPORT;
        default: return HCCL_SUCCESS;
    }
}

HcclResult CheckReduceOp(const char* opName, HcclDataType t, HcclReduceOp op)
{
    if ((int)op < 0 || op >= HCCL_REDUCE_RESERVED) {
        ReportInputError("EI0003", opName, "op", std::to_string((int)op), "sum, prod, max or min");
        return HCCL_E_PARA;
    }
    if (op == HCCL_REDUCE_PROD) {
        switch (t) {
            case HCCL_DATA_TYPE_INT8: case HCCL_DATA_TYPE_INT32: case HCCL_DATA_TYPE_INT64: case HCCL_DATA_TYPE_UINT64:
            case HCCL_DATA_TYPE_FP16: case HCCL_DATA_TYPE_FP32: case HCCL_DATA_TYPE_FP64: break;
            default:
                ReportInputError("EI0003", opName, "op", "prod", "prod is defined for int8, int32, int64, uint64, float16, float32, float64");
                return HCCL_E_NOT_SUPPORT;
        }
    }
    if ((t == HCCL_DATA_TYPE_FP8E4M3 || t == HCCL_DATA_TYPE_FP8E5M2) && op != HCCL_REDUCE_SUM && op != HCCL_REDUCE_MAX && op != HCCL_REDUCE_MIN)
        return HCCL_E_NOT_SUPPORT;
    return HCCL_SUCCESS;
}

HcclResult CheckRank(const char* opName, const char* what, uint32_t rank, uint32_t rankSize)
{
    if (rank >= rankSize) {
        ReportInputError("EI0003", opName, what, std::to_string(rank), ("a rank below " + std::to_string(rankSize)).c_str());
        return HCCL_E_PARA;
    }
    return HCCL_SUCCESS;
}

HcclResult CheckGroupName(const std::string& name)
{
    if (name.empty() || name.size() > kGroupNameMaxLen) { HCCL_ERROR("group name must have 1..%u characters (got %zu)", kGroupNameMaxLen, name.size()); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}
HcclResult CheckTag(const std::string& tag)
{
    if (tag.empty() || tag.size() > 255) { HCCL_ERROR("tag must have 1..255 characters (got %zu)", tag.size()); return HCCL_E_PARA; }
    return HCCL_SUCCESS;
}

}  // namespace hccl
