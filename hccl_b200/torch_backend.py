"""``torch.distributed`` backend "hccl": collectives of this library behind the stock PyTorch API.

    import hccl_b200.torch_backend            # registers the backend
    dist.init_process_group("hccl", rank=rank, world_size=world, store=store)   # or init_method / env://
    dist.all_reduce(t)                        # runs HcclAllReduce on the current CUDA stream

Counterpart of the reference's PyTorch example, which wraps hccl4py calls in a helper class
(experimental/eco_system/python/examples/03_pytorch_integration/allreduce_test.py) - here the binding is a
real process-group backend, so unmodified ``torch.distributed`` code runs on it.

Operators are enqueued on the caller's current stream and return an already-completed work object (stream-ordered
semantics, like NCCL's with ``async_op=False``).  The root info travels through the group's store.
"""
from __future__ import annotations

from datetime import timedelta

import torch
import torch.distributed as dist

from .comm import Communicator
from .types import ReduceOp

_REDUCE = {dist.ReduceOp.SUM: ReduceOp.SUM, dist.ReduceOp.PRODUCT: ReduceOp.PROD, dist.ReduceOp.MAX: ReduceOp.MAX,
           dist.ReduceOp.MIN: ReduceOp.MIN}


def _is_avg(op) -> bool:
    key = getattr(op, "op", op) if not isinstance(op, dist.ReduceOp.RedOpType) else op
    return key == dist.ReduceOp.AVG


def _red(op) -> ReduceOp:
    # torch passes either the enum value or a ReduceOp object wrapping it
    key = getattr(op, "op", op) if not isinstance(op, dist.ReduceOp.RedOpType) else op
    if key == dist.ReduceOp.AVG:
        return ReduceOp.SUM              # the caller scales by 1 / world inside the same kernel (all_reduce_ex)
    for k, v in _REDUCE.items():
        if key == k:
            return v
    raise NotImplementedError(f"hccl backend: reduce op {op} is not supported (sum, avg, prod, max, min are)")


class _DoneWork(dist._Work):
    """Work handle of a stream-ordered operator: the kernel is in the stream, there is nothing to wait for on the host."""

    def __init__(self, result=None):
        super().__init__()
        self._result = result
        self._future = torch.futures.Future()
        self._future.set_result(result)

    def wait(self, timeout=None):
        return True

    def is_completed(self):
        return True

    def is_success(self):
        return True

    def get_future(self):
        return self._future

    def result(self):
        return self._result


class ProcessGroupHCCL(dist.ProcessGroup):
    def __init__(self, store, rank: int, size: int, timeout: timedelta | None = None, config=None):
        super().__init__(rank, size)
        self._rank, self._size = rank, size
        if rank == 0:
            info = Communicator.get_root_info()
            store.set("hccl_root_info", info)
        else:
            info = bytes(store.get("hccl_root_info"))
        self.comm = Communicator.from_root_info(info, rank, size, config=config)
        self._store = store

    # ---- identification
    def getBackendName(self):
        return "hccl"

    def name(self):
        return "hccl"

    def rank(self):
        return self._rank

    def size(self):
        return self._size

    # ---- collectives
    def allreduce(self, tensors, opts=None):
        op = _red(opts.reduceOp) if opts is not None else ReduceOp.SUM
        avg = opts is not None and _is_avg(opts.reduceOp)
        for t in tensors:
            if avg and t.dtype in (torch.float32, torch.bfloat16, torch.float16) and self._size > 1:
                self.comm.all_reduce_ex(self._c(t), scale=1.0 / self._size)          # the average is fused into the reduction
            else:
                self.comm.all_reduce(self._c(t), op=op)
                if avg:
                    t.div_(self._size)
        return _DoneWork(tensors)

    def allreduce_coalesced(self, tensors, opts=None):
        return self.allreduce(tensors, opts)

    def broadcast(self, tensors, opts=None):
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            self.comm.broadcast(self._c(t), root)
        return _DoneWork(tensors)

    def reduce(self, tensors, opts=None):
        op = _red(opts.reduceOp) if opts is not None else ReduceOp.SUM
        root = opts.rootRank if opts is not None else 0
        for t in tensors:
            t = self._c(t)
            out = t if self._rank == root else torch.empty_like(t)
            self.comm.reduce(t, out, root, op)
        return _DoneWork(tensors)

    def _allgather_base(self, output, input, opts=None):
        self.comm.all_gather(self._c(input), self._c(output))
        return _DoneWork(output)

    def allgather(self, output_tensors, input_tensors, opts=None):
        for outs, inp in zip(output_tensors, input_tensors):
            flat = torch.empty((self._size,) + tuple(inp.shape), device=inp.device, dtype=inp.dtype)
            self.comm.all_gather(self._c(inp), flat)
            for q, o in enumerate(outs):
                o.copy_(flat[q])
        return _DoneWork(output_tensors)

    def allgather_into_tensor_coalesced(self, outputs, inputs, opts=None):
        for o, i in zip(outputs, inputs):
            self.comm.all_gather(self._c(i), self._c(o))
        return _DoneWork(outputs)

    def _reduce_scatter_base(self, output, input, opts=None):
        op = _red(opts.reduceOp) if opts is not None else ReduceOp.SUM
        if opts is not None and _is_avg(opts.reduceOp) and self._size > 1:
            if input.dtype in (torch.float32, torch.bfloat16, torch.float16):
                self.comm.reduce_scatter_ex(self._c(input), self._c(output), scale=1.0 / self._size)
            else:
                self.comm.reduce_scatter(self._c(input), self._c(output), op)
                output.div_(self._size)
            return _DoneWork(output)
        self.comm.reduce_scatter(self._c(input), self._c(output), op)
        return _DoneWork(output)

    def reduce_scatter(self, output_tensors, input_tensors, opts=None):
        op = _red(opts.reduceOp) if opts is not None else ReduceOp.SUM
        for out, ins in zip(output_tensors, input_tensors):
            flat = torch.stack([i.contiguous() for i in ins])
            self.comm.reduce_scatter(flat, self._c(out), op)
        return _DoneWork(output_tensors)

    def reduce_scatter_tensor_coalesced(self, outputs, inputs, opts=None):
        op = _red(opts.reduceOp) if opts is not None else ReduceOp.SUM
        for o, i in zip(outputs, inputs):
            self.comm.reduce_scatter(self._c(i), self._c(o), op)
        return _DoneWork(outputs)

    def alltoall_base(self, output, input, output_split_sizes, input_split_sizes, opts=None):
        if not output_split_sizes and not input_split_sizes:
            self.comm.all_to_all(self._c(input), self._c(output))
            return _DoneWork(output)
        row = input[0].numel() if input.dim() > 1 else 1
        sc = [int(s) * row for s in input_split_sizes]
        rc = [int(s) * row for s in output_split_sizes]
        sd = [sum(sc[:q]) for q in range(self._size)]
        rd = [sum(rc[:q]) for q in range(self._size)]
        self.comm.all_to_all_v(self._c(input), sc, sd, self._c(output), rc, rd)
        return _DoneWork(output)

    def alltoall(self, output_tensors, input_tensors, opts=None):
        sc = [t.numel() for t in input_tensors]
        rc = [t.numel() for t in output_tensors]
        sd = [sum(sc[:q]) for q in range(self._size)]
        rd = [sum(rc[:q]) for q in range(self._size)]
        send = torch.cat([t.reshape(-1) for t in input_tensors])
        recv = torch.empty(sum(rc), device=send.device, dtype=send.dtype)
        self.comm.all_to_all_v(send, sc, sd, recv, rc, rd)
        for q, o in enumerate(output_tensors):
            o.copy_(recv[rd[q]:rd[q] + rc[q]].view_as(o))
        return _DoneWork(output_tensors)

    def scatter(self, output_tensors, input_tensors, opts=None):
        root = opts.rootRank if opts is not None else 0
        for i, out in enumerate(output_tensors):
            send = torch.stack([t.contiguous() for t in input_tensors[i]]) if self._rank == root else None
            self.comm.scatter(send, self._c(out), root)
        return _DoneWork(output_tensors)

    def gather(self, output_tensors, input_tensors, opts=None):
        root = opts.rootRank if opts is not None else 0
        for i, inp in enumerate(input_tensors):
            flat = torch.empty((self._size,) + tuple(inp.shape), device=inp.device, dtype=inp.dtype)
            self.comm.all_gather(self._c(inp), flat)      # the library has no Gather operator (neither has the reference)
            if self._rank == root:
                for q, o in enumerate(output_tensors[i]):
                    o.copy_(flat[q])
        return _DoneWork(output_tensors)

    def send(self, tensors, dst, tag=0):
        for t in tensors:
            self.comm.send(self._c(t), dst)
        return _DoneWork(None)

    def recv(self, tensors, src, tag=0):
        for t in tensors:
            self.comm.recv(self._c(t), src)
        return _DoneWork(None)

    def barrier(self, opts=None):
        self.comm.barrier()
        torch.cuda.current_stream().synchronize()
        return _DoneWork(None)

    def shutdown(self):
        if self.comm is not None:
            self.comm.destroy()
            self.comm = None

    def abort(self):
        self.shutdown()

    @staticmethod
    def _c(t):
        if not t.is_contiguous():
            raise ValueError("hccl backend: tensors must be contiguous")
        return t


def _create(store, rank, size, timeout):
    return ProcessGroupHCCL(store, rank, size, timeout)


def register() -> None:
    """Idempotent registration of the "hccl" backend for CUDA tensors."""
    if "HCCL" not in dist.Backend._plugins:
        dist.Backend.register_backend("hccl", _create, devices=["cuda"])


register()
