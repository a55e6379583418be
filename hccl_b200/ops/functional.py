"""torch.distributed-style functional collectives on a default communicator.

    import hccl_b200.ops.functional as hdist
    hdist.init_process_group()            # after torch.distributed.init_process_group(...)
    hdist.all_reduce(t)                   # in place, like torch.distributed.all_reduce

Signatures follow ``torch.distributed`` (tensor first, ``op``, ``async_op`` is
accepted and ignored: every call is asynchronous on the current CUDA stream and
ordered with the kernels around it, as NCCL calls are).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..comm import Communicator
from ..types import ReduceOp

_default: Optional[Communicator] = None


def init_process_group(config=None, group=None) -> Communicator:
    global _default
    _default = Communicator.from_torch_distributed(group=group, config=config)
    return _default


def destroy_process_group():
    global _default
    if _default is not None:
        _default.destroy()
        _default = None


def get_communicator() -> Communicator:
    if _default is None:
        raise RuntimeError("call hccl_b200.ops.functional.init_process_group() first")
    return _default


def get_rank() -> int:
    return get_communicator().rank


def get_world_size() -> int:
    return get_communicator().world_size


def _op(op) -> ReduceOp:
    if isinstance(op, ReduceOp):
        return op
    name = str(op).split(".")[-1].upper()
    return {"SUM": ReduceOp.SUM, "PRODUCT": ReduceOp.PROD, "PROD": ReduceOp.PROD, "MAX": ReduceOp.MAX, "MIN": ReduceOp.MIN}[name]


def all_reduce(tensor, op=ReduceOp.SUM, async_op=False):
    get_communicator().all_reduce(tensor, tensor, _op(op))


def broadcast(tensor, src=0, async_op=False):
    get_communicator().broadcast(tensor, src)


def reduce(tensor, dst=0, op=ReduceOp.SUM, async_op=False):
    c = get_communicator()
    c.reduce(tensor, tensor if c.rank == dst else None, dst, _op(op))


def all_gather_into_tensor(output, input, async_op=False):
    get_communicator().all_gather(input, output)


def all_gather(tensor_list: List[torch.Tensor], tensor, async_op=False):
    out = torch.empty((len(tensor_list),) + tuple(tensor.shape), dtype=tensor.dtype, device=tensor.device)
    get_communicator().all_gather(tensor.contiguous(), out)
    for i, t in enumerate(tensor_list):
        t.copy_(out[i])


def reduce_scatter_tensor(output, input, op=ReduceOp.SUM, async_op=False):
    get_communicator().reduce_scatter(input, output, _op(op))


def scatter(tensor, scatter_list=None, src=0, async_op=False):
    c = get_communicator()
    send = torch.stack([t.contiguous() for t in scatter_list]).contiguous() if c.rank == src else None
    c.scatter(send, tensor, src)


def all_to_all_single(output, input, output_split_sizes=None, input_split_sizes=None, async_op=False):
    c = get_communicator()
    if output_split_sizes is None and input_split_sizes is None:
        c.all_to_all(input, output)
        return
    row = input[0].numel() if input.dim() > 1 else 1
    sc = [s * row for s in input_split_sizes]
    rc = [s * row for s in output_split_sizes]
    sd = [sum(sc[:i]) for i in range(len(sc))]
    rd = [sum(rc[:i]) for i in range(len(rc))]
    c.all_to_all_v(input, sc, sd, output, rc, rd)


def send(tensor, dst, async_op=False):
    get_communicator().send(tensor, dst)


def recv(tensor, src, async_op=False):
    get_communicator().recv(tensor, src)


def batch_isend_irecv(ops):
    """ops: list of ("send" | "recv", tensor, peer)."""
    get_communicator().batch_send_recv(ops)


def barrier(async_op=False):
    get_communicator().barrier()
