"""hccl_b200: a Blackwell-native collective communication library with the
HCCL operator set.

Layers: :mod:`hccl_b200._lib` (ctypes over ``libhccl_b200.so``),
:mod:`hccl_b200.comm` (communicators and operators on tensors),
:mod:`hccl_b200.ops` (torch.distributed-style functional API, MC2 fused
matmul+collective ops, MoE dispatch / combine), :mod:`hccl_b200.parallel`
(process-group binding, tensor/sequence-parallel layers),
:mod:`hccl_b200.models` (the TP+SP decoder used by the benchmark) and
:mod:`hccl_b200.utils`.
"""
from .types import Cmd, CommStatus, DataType, Engine, HcclError, ReduceOp, Result  # noqa: F401
from .comm import Communicator, registry  # noqa: F401
from ._lib import make_config  # noqa: F401

__version__ = "0.1.0"
