"""ctypes binding of ``libhccl_b200.so`` (the role of hccl4py's ctypes layer,
reference ``experimental/eco_system/python/hccl4py/ops.py:50-499``).

The shared object is built in-tree by :mod:`hccl_b200.build`.  It is loaded on
import; when it is missing it is built if a compiler is present, otherwise the
import fails loudly - there is no pure-Python fallback for any operator.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_double, c_int, c_int32, c_uint8, c_uint32, c_uint64, c_void_p
from pathlib import Path

# HCCL_B200_LIB names another build of the library (the AddressSanitizer variant of `build.py --asan`)
_LIB_PATH = Path(os.environ["HCCL_B200_LIB"]) if os.environ.get("HCCL_B200_LIB") else Path(__file__).resolve().parent / "lib" / "libhccl_b200.so"


def _load() -> ctypes.CDLL:
    if not _LIB_PATH.exists() or os.environ.get("HCCL_B200_REBUILD") == "1":
        from . import build as _build

        _build.build()
    return ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)


lib = _load()

HCCL_ROOT_INFO_BYTES = 4108


class HcclRootInfo(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_char * HCCL_ROOT_INFO_BYTES)]


class HcclCommConfig(ctypes.Structure):
    _fields_ = [
        ("size", c_uint32), ("magicWord", c_uint32), ("version", c_uint32), ("reserved", c_uint32),
        ("hcclBufferSize", c_uint32), ("hcclDeterministic", c_uint32), ("hcclCommName", ctypes.c_char * 128),
        ("hcclOpExpansionMode", c_uint32), ("hcclExecTimeoutMs", c_uint32), ("hcclMaxBlocks", c_uint32),
        ("hcclNvlsEnable", c_uint32), ("padding", ctypes.c_char * (2304 - 16 - 8 - 128 - 16)),
    ]


assert ctypes.sizeof(HcclCommConfig) == 2304


class HcclSendRecvItem(ctypes.Structure):
    _fields_ = [("sendRecvType", c_int), ("buf", c_void_p), ("count", c_uint64), ("dataType", c_int), ("remoteRank", c_uint32)]


def make_config(buffer_mib: int = 0, deterministic: int | None = None, name: str = "", engine: int = 0,
                exec_timeout_ms: int = 0, max_blocks: int = 0, nvls: int = 0) -> HcclCommConfig:
    cfg = HcclCommConfig()
    cfg.size = ctypes.sizeof(HcclCommConfig)
    cfg.magicWord = 0xF0F0F0F0
    cfg.version = 1
    cfg.hcclBufferSize = buffer_mib
    cfg.hcclDeterministic = 0xFFFFFFFF if deterministic is None else int(deterministic)
    cfg.hcclCommName = name.encode()[:127]
    cfg.hcclOpExpansionMode = engine
    cfg.hcclExecTimeoutMs = exec_timeout_ms
    cfg.hcclMaxBlocks = max_blocks
    cfg.hcclNvlsEnable = nvls
    return cfg


def _sig(name, restype, *argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = list(argtypes)
    return fn


R = c_int  # HcclResult
_sig("HcclGetRootInfo", R, POINTER(HcclRootInfo))
_sig("HcclCommInitRootInfo", R, c_uint32, POINTER(HcclRootInfo), c_uint32, POINTER(c_void_p))
_sig("HcclCommInitRootInfoConfig", R, c_uint32, POINTER(HcclRootInfo), c_uint32, POINTER(HcclCommConfig), POINTER(c_void_p))
_sig("HcclCommInitClusterInfo", R, c_char_p, c_uint32, POINTER(c_void_p))
_sig("HcclCommInitClusterInfoConfig", R, c_char_p, c_uint32, POINTER(HcclCommConfig), POINTER(c_void_p))
_sig("HcclCommInitAll", R, c_uint32, POINTER(c_int32), POINTER(c_void_p))
_sig("HcclCommInitEmulated", R, c_uint32, POINTER(HcclCommConfig), POINTER(c_void_p))
_sig("HcclCommInitHostSim", R, c_uint32, c_char_p, POINTER(HcclCommConfig), POINTER(c_void_p))
_sig("HcclCommDestroy", R, c_void_p)
_sig("HcclGetRankSize", R, c_void_p, POINTER(c_uint32))
_sig("HcclGetRankId", R, c_void_p, POINTER(c_uint32))
_sig("HcclGetCommName", R, c_void_p, c_char_p)
_sig("HcclCommGetStatus", R, c_void_p, POINTER(c_int))
_sig("HcclCommSuspend", R, c_void_p)
_sig("HcclCommResume", R, c_void_p)
_sig("HcclCommGetAsyncError", R, c_void_p, POINTER(c_int))
_sig("HcclGetErrorString", c_char_p, c_int)
_sig("HcclGetHcclBuffer", R, c_void_p, POINTER(c_void_p), POINTER(c_uint64))
_sig("HcclMemAlloc", R, c_void_p, c_uint64, POINTER(c_void_p))
_sig("HcclMemFree", R, c_void_p, c_void_p)
_sig("HcclCommSymWinGet", R, c_void_p, c_void_p, c_uint32, POINTER(c_void_p))
_sig("HcclCommSymWinGetMulticast", R, c_void_p, c_void_p, POINTER(c_void_p))
_sig("HcclAllReduce", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_void_p, c_void_p)
_sig("HcclAllReduceEx", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_int, ctypes.c_float, c_void_p, c_void_p)
_sig("HcclReduceScatterEx", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_int, ctypes.c_float, c_void_p, c_void_p)
_sig("HcclBroadcast", R, c_void_p, c_uint64, c_int, c_uint32, c_void_p, c_void_p)
_sig("HcclReduceScatter", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_void_p, c_void_p)
_sig("HcclReduceScatterV", R, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_int, c_int, c_void_p, c_void_p)
_sig("HcclScatter", R, c_void_p, c_void_p, c_uint64, c_int, c_uint32, c_void_p, c_void_p)
_sig("HcclAllGather", R, c_void_p, c_void_p, c_uint64, c_int, c_void_p, c_void_p)
_sig("HcclAllGatherV", R, c_void_p, c_uint64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p)
_sig("HcclSend", R, c_void_p, c_uint64, c_int, c_uint32, c_void_p, c_void_p)
_sig("HcclRecv", R, c_void_p, c_uint64, c_int, c_uint32, c_void_p, c_void_p)
_sig("HcclAlltoAllVC", R, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p)
_sig("HcclAlltoAllV", R, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p)
_sig("HcclAlltoAll", R, c_void_p, c_uint64, c_int, c_void_p, c_uint64, c_int, c_void_p, c_void_p)
_sig("HcclReduce", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_uint32, c_void_p, c_void_p)
_sig("HcclBatchSendRecv", R, POINTER(HcclSendRecvItem), c_uint32, c_void_p, c_void_p)
_sig("HcclBarrier", R, c_void_p, c_void_p)
# extensions
_sig("HcclGetLastAlgName", R, c_void_p, c_char_p, c_uint32)
_sig("HcclSelectorExplain", R, c_void_p, c_int, c_uint64, c_int, c_int, c_int, c_char_p, c_uint32)
_sig("HcclAlgRegistryCount", c_uint32)
_sig("HcclAlgRegistryEntry", R, c_uint32, c_char_p, c_uint32, POINTER(c_int), POINTER(c_int))
_sig("HcclProfilingSetLevel", R, c_int)
_sig("HcclProfilingDump", R, c_char_p, c_uint32)
_sig("HcclHostTraceBegin", R, c_void_p)
_sig("HcclHostTraceVerify", R, c_void_p, c_char_p, c_uint32)
_sig("HcclTestLaunchUnsignalledWait", R, c_void_p, c_void_p)
_sig("HcclTestInjectBootstrapFailure", R, c_void_p)
_sig("HcclTestHostDropPosts", R, c_void_p, ctypes.c_uint32)
_sig("HcclTestHostRecoveries", R, c_void_p, ctypes.POINTER(ctypes.c_uint64))
_sig("HcclGetPlanCacheStats", R, c_void_p, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64))
_sig("HcclSetLinkModel", R, c_double, c_double, c_double, c_double, c_double, c_double)
_sig("HcclGetVersion", c_char_p)
_sig("HcclReloadEnvConfig", R)
# MC2
_sig("HcclKfcAllocOpArgs", R, POINTER(c_void_p))
_sig("HcclKfcFreeOpArgs", R, c_void_p)
_sig("HcclKfcOpArgsSetSrcDataType", R, c_void_p, c_uint8)
_sig("HcclKfcOpArgsSetDstDataType", R, c_void_p, c_uint8)
_sig("HcclKfcOpArgsSetReduceType", R, c_void_p, c_uint32)
_sig("HcclKfcOpArgsSetCount", R, c_void_p, c_uint64)
_sig("HcclKfcOpArgsSetAlgConfig", R, c_void_p, c_char_p)
_sig("HcclKfcOpArgsSetCommEngine", R, c_void_p, c_uint8)
_sig("HcclCreateOpResCtx", R, c_void_p, c_uint8, c_void_p, POINTER(c_void_p))
_sig("HcclMc2Matmul", R, c_void_p, c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, c_int, c_int, c_void_p)
_sig("HcclMc2AllGatherMatmul", R, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, c_int, c_void_p, c_void_p)
_sig("HcclMc2MatmulReduceScatter", R, c_void_p, c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, c_int, c_void_p, c_void_p)
_sig("HcclMc2MatmulAllReduce", R, c_void_p, c_void_p, c_void_p, c_uint64, c_uint64, c_uint64, c_int, c_void_p, c_void_p)
# fused element-wise kernels of the decoder stack


def _sig_or_none(name, restype, *argtypes):
    """Like _sig for entry points added after the first release of the ABI: None when the loaded library predates them
    (callers raise a clear error instead of the import failing)."""
    try:
        return _sig(name, restype, *argtypes)
    except AttributeError:
        return None


_sig_or_none("HcclFusedAddRmsNormFwd", R, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, ctypes.c_float, c_void_p)
_sig_or_none("HcclFusedRmsNormBwdPartials", c_uint32, c_uint64)
_sig_or_none("HcclFusedRmsNormBwd", R, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_void_p)
_sig_or_none("HcclFusedSwigluFwd", R, c_void_p, c_void_p, c_uint64, c_uint32, c_void_p)
_sig_or_none("HcclFusedSwigluBwd", R, c_void_p, c_void_p, c_void_p, c_uint64, c_uint32, c_void_p)
_sig_or_none("HcclFusedRope", R, c_void_p, c_uint64, c_void_p, c_uint64, c_void_p, c_void_p, c_uint64, c_uint32, c_uint32, c_int, c_void_p)
_sig_or_none("HcclCommRegister", R, c_void_p, c_void_p, c_uint64)
_sig_or_none("HcclCommDeregister", R, c_void_p, c_void_p)
# MoE
class HcclMoeConfig(ctypes.Structure):
    _fields_ = [("nTokens", c_uint32), ("hidden", c_uint32), ("topk", c_uint32), ("nExperts", c_uint32), ("capacity", c_uint32)]


_sig("HcclMoeDispatch", R, c_void_p, c_void_p, c_void_p, POINTER(HcclMoeConfig), c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p)
_sig("HcclMoeCombine", R, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(HcclMoeConfig), c_void_p, c_void_p)
_sig("HcclMoeExpertOffsets", R, c_void_p, c_uint64, c_uint32, c_void_p, c_void_p)
_sig("HcclDebugStepTable", R, c_char_p, c_uint32, c_uint32, c_char_p, c_char_p, c_uint32)
_sig("HcclDebugParseEnv", R, c_char_p, c_char_p, c_uint32)
_sig("HcclDebugEvalCost", c_double, c_double, c_double, c_double, c_double, c_int, c_double, c_double)


class HcclOpResource(ctypes.Structure):
    _fields_ = [("algName", ctypes.c_char * 128), ("engine", c_uint32), ("blocks", c_uint32), ("launches", c_uint32), ("streams", c_uint32),
                ("scratchBytes", c_uint64)]


_sig("HcclCalcOpResource", R, c_void_p, c_int, c_uint64, c_int, c_int, c_int, POINTER(HcclOpResource))


if hasattr(lib, "HcclDiagnoseDump"):
    _sig("HcclDiagnoseDump", R, ctypes.c_char_p, c_uint32)
if hasattr(lib, "HcclFusedAdamW"):
    _sig("HcclFusedAdamW", R, c_void_p, c_uint32, c_int, c_int, ctypes.c_float, c_void_p, ctypes.c_float, ctypes.c_float, ctypes.c_float,
         ctypes.c_float, c_void_p, c_void_p)
    _sig("HcclFusedAdamWLaunches", c_uint32, c_uint32)


class HcclResPackGraphMode(ctypes.Structure):
    _fields_ = [("size", c_uint32), ("scratch", c_void_p), ("scratchBytes", c_uint64), ("slaveStreams", POINTER(c_void_p)),
                ("slaveStreamNum", c_uint32)]


# graph-mode twins: the group is named, not passed as a handle (hccl_graph_mode.h)
_RP = POINTER(HcclResPackGraphMode)
_sig("HcclGroupGetComm", R, c_char_p, POINTER(c_void_p))
_sig("HcclGroupBindThread", R, c_void_p)
_sig("HcclGroupUnbindThread", R, c_char_p)
_sig("HcclCalcOpResGraphMode", R, c_char_p, c_int, c_uint64, c_int, c_int, POINTER(HcclOpResource))
_sig("HcclAllReduceGraphMode", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclBroadcastGraphMode", R, c_void_p, c_uint64, c_int, c_uint32, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclReduceScatterGraphMode", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclAllGatherGraphMode", R, c_void_p, c_void_p, c_uint64, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclReduceGraphMode", R, c_void_p, c_void_p, c_uint64, c_int, c_int, c_uint32, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclScatterGraphMode", R, c_void_p, c_void_p, c_uint64, c_int, c_uint32, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclAlltoAllGraphMode", R, c_void_p, c_uint64, c_int, c_void_p, c_uint64, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclSendGraphMode", R, c_void_p, c_uint64, c_int, c_uint32, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclRecvGraphMode", R, c_void_p, c_uint64, c_int, c_uint32, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclBarrierGraphMode", R, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclAllGatherVGraphMode", R, c_void_p, c_void_p, c_uint64, c_void_p, c_void_p, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclReduceScatterVGraphMode", R, c_void_p, c_void_p, c_void_p, c_void_p, c_uint64, c_int, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclAlltoAllVGraphMode", R, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclAlltoAllVCGraphMode", R, c_void_p, c_void_p, c_int, c_void_p, c_int, c_char_p, c_char_p, _RP, c_void_p)
_sig("HcclCreateOpParamGraphMode", R, POINTER(c_void_p))
_sig("HcclDestroyOpParamGraphMode", R, c_void_p)
_sig("HcclSetOpParamGraphModeOpType", R, c_void_p, c_char_p)
_sig("HcclSetOpParamGraphModeDataCount", R, c_void_p, c_uint64)
_sig("HcclSetOpParamGraphModeRankSize", R, c_void_p, c_uint32)
_sig("HcclSetOpParamGraphModeHCCLBufferSize", R, c_void_p, c_uint64)
_sig("HcclSetOpParamGraphModeDataType", R, c_void_p, c_int)
_sig("HcclSetOpParamGraphModeReduceType", R, c_void_p, c_int)
_sig("HcclSetOpParamGraphModeRegistered", R, c_void_p, c_int, c_int)
_sig("HcclSetOpParamGraphModeBlockLimit", R, c_void_p, c_uint32)
_sig("HcclCalcOpResOpParamGraphMode", R, c_void_p, POINTER(c_uint64), POINTER(c_uint32), POINTER(c_uint32), POINTER(c_uint32), c_char_p)
_sig("HcclSelectAlgGraphMode", R, c_char_p, c_uint64, c_int, c_int, c_int, c_uint32, POINTER(ctypes.c_bool), c_char_p)
_sig("HcclCalcBlockNumGraphMode", R, c_char_p, c_uint64, c_int, c_int, c_int, c_uint32, POINTER(c_uint32))
_sig("HcclGetAlgExecParamGraphMode", R, c_char_p, c_char_p, c_uint64, c_int, c_int, c_int, POINTER(c_void_p), POINTER(c_uint64))
_sig("HcclSetBlockLimitGraphMode", R, c_char_p, c_uint32)
_sig("HcclAlgoPluginQueryAlgs", R, c_char_p, c_char_p, c_uint32, POINTER(c_uint32))
_sig("HcclCalcOpResOnlineGraphMode", R, c_char_p, c_int, c_uint64, c_int, c_int, c_int, POINTER(HcclOpResource))
_sig("HcclCalcOpResOfflineGraphMode", R, c_uint32, c_int, c_uint64, c_int, c_uint64, c_int, c_int, c_int, POINTER(HcclOpResource))
