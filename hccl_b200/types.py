"""Enumerations of the C API and the mapping to torch / numpy dtypes."""
from __future__ import annotations

import enum


class Result(enum.IntEnum):
    SUCCESS = 0
    E_PARA = 1
    E_PTR = 2
    E_MEMORY = 3
    E_INTERNAL = 4
    E_NOT_SUPPORT = 5
    E_NOT_FOUND = 6
    E_UNAVAIL = 7
    E_SYSCALL = 8
    E_TIMEOUT = 9
    E_OPEN_FILE_FAILURE = 10
    E_TCP_CONNECT = 11
    E_ROCE_CONNECT = 12
    E_TCP_TRANSFER = 13
    E_ROCE_TRANSFER = 14
    E_RUNTIME = 15
    E_DRV = 16
    E_PROFILING = 17
    E_CCE = 18
    E_NETWORK = 19
    E_AGAIN = 20
    E_REMOTE = 21
    E_SUSPENDING = 22
    E_OPRETRY_FAIL = 23
    E_OOM = 24


class ReduceOp(enum.IntEnum):
    SUM = 0
    PROD = 1
    MAX = 2
    MIN = 3


class DataType(enum.IntEnum):
    INT8 = 0
    INT16 = 1
    INT32 = 2
    FP16 = 3
    FP32 = 4
    INT64 = 5
    UINT64 = 6
    UINT8 = 7
    UINT16 = 8
    UINT32 = 9
    FP64 = 10
    BFP16 = 11
    INT128 = 12
    HIF8 = 14
    FP8E4M3 = 15
    FP8E5M2 = 16
    FP8E8M0 = 17


class Cmd(enum.IntEnum):
    BROADCAST = 1
    ALLREDUCE = 2
    REDUCE = 3
    SEND = 4
    RECEIVE = 5
    ALLGATHER = 6
    REDUCE_SCATTER = 7
    ALLTOALLV = 8
    ALLTOALLVC = 9
    ALLTOALL = 10
    GATHER = 11
    SCATTER = 12
    BATCH_SEND_RECV = 13
    ALLGATHER_V = 16
    REDUCE_SCATTER_V = 17
    BARRIER = 18


class Engine(enum.IntEnum):
    AUTO = 0
    P2P = 1
    NVLS = 2
    HOSTCPU = 3


class CommStatus(enum.IntEnum):
    READY = 0
    SUSPENDING = 1
    ERROR = 2
    DESTROYED = 3


DTYPE_SIZE = {
    DataType.INT8: 1, DataType.UINT8: 1, DataType.HIF8: 1, DataType.FP8E4M3: 1, DataType.FP8E5M2: 1, DataType.FP8E8M0: 1,
    DataType.INT16: 2, DataType.UINT16: 2, DataType.FP16: 2, DataType.BFP16: 2,
    DataType.INT32: 4, DataType.UINT32: 4, DataType.FP32: 4,
    DataType.INT64: 8, DataType.UINT64: 8, DataType.FP64: 8, DataType.INT128: 16,
}


_TORCH_MAP = None
_NUMPY_MAP = None


def torch_dtype_map():
    """torch dtype -> DataType (built once: operators look it up on every call)."""
    global _TORCH_MAP
    if _TORCH_MAP is not None:
        return _TORCH_MAP
    import torch

    m = {
        torch.int8: DataType.INT8, torch.int16: DataType.INT16, torch.int32: DataType.INT32, torch.float16: DataType.FP16,
        torch.float32: DataType.FP32, torch.int64: DataType.INT64, torch.uint8: DataType.UINT8, torch.float64: DataType.FP64,
        torch.bfloat16: DataType.BFP16, torch.bool: DataType.UINT8,
    }
    for name, dt in (("uint16", DataType.UINT16), ("uint32", DataType.UINT32), ("uint64", DataType.UINT64),
                     ("float8_e4m3fn", DataType.FP8E4M3), ("float8_e5m2", DataType.FP8E5M2)):
        if hasattr(torch, name):
            m[getattr(torch, name)] = dt
    _TORCH_MAP = m
    return m


def numpy_dtype_map():
    global _NUMPY_MAP
    if _NUMPY_MAP is not None:
        return _NUMPY_MAP
    import numpy as np

    _NUMPY_MAP = {
        np.dtype(np.int8): DataType.INT8, np.dtype(np.int16): DataType.INT16, np.dtype(np.int32): DataType.INT32,
        np.dtype(np.float16): DataType.FP16, np.dtype(np.float32): DataType.FP32, np.dtype(np.int64): DataType.INT64,
        np.dtype(np.uint64): DataType.UINT64, np.dtype(np.uint8): DataType.UINT8, np.dtype(np.uint16): DataType.UINT16,
        np.dtype(np.uint32): DataType.UINT32, np.dtype(np.float64): DataType.FP64,
    }
    return _NUMPY_MAP


class HcclError(RuntimeError):
    def __init__(self, code: int, what: str):
        self.code = Result(code) if code in Result._value2member_map_ else code
        super().__init__(f"{what} failed: {self.code!r}")
