"""Python communicator over the C API.

A :class:`Communicator` wraps one ``HcclComm``.  Device communicators take CUDA
``torch.Tensor`` arguments and run on the current CUDA stream; host-engine
communicators (simulated ranks) take ``numpy`` arrays.  Creation paths mirror
the C API: root-info rendezvous (one process per GPU), rank table, emulated
ranks on one GPU, and host-simulated ranks.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_uint32, c_uint64, c_void_p
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import lib
from .types import Cmd, CommStatus, DataType, HcclError, ReduceOp, Result, numpy_dtype_map, torch_dtype_map


def _check(code: int, what: str) -> None:
    if code != 0:
        raise HcclError(code, what)


class _CudaBuffer:
    """Exposes raw device memory through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _u64_array(values: Sequence[int]):
    return (c_uint64 * len(values))(*[int(v) for v in values])


class Communicator:
    def __init__(self, handle: int, kind: str, keepalive=None):
        self._h = c_void_p(handle)
        self.kind = kind  # "device" | "emulated" | "host"
        self._keep = keepalive
        n, r = c_uint32(), c_uint32()
        _check(lib.HcclGetRankSize(self._h, byref(n)), "HcclGetRankSize")
        _check(lib.HcclGetRankId(self._h, byref(r)), "HcclGetRankId")
        self.world_size, self.rank = n.value, r.value
        self._sym = []  # symmetric allocations (ptr, nbytes)

    # ------------------------------------------------------------------ creation
    @staticmethod
    def get_root_info() -> bytes:
        info = _lib.HcclRootInfo()
        _check(lib.HcclGetRootInfo(byref(info)), "HcclGetRootInfo")
        return ctypes.string_at(ctypes.addressof(info), ctypes.sizeof(info))

    @classmethod
    def from_root_info(cls, root_info: bytes, rank: int, world_size: int, config: Optional[_lib.HcclCommConfig] = None):
        info = _lib.HcclRootInfo()
        ctypes.memmove(ctypes.addressof(info), root_info, min(len(root_info), ctypes.sizeof(info)))
        h = c_void_p()
        if config is None:
            _check(lib.HcclCommInitRootInfo(world_size, byref(info), rank, byref(h)), "HcclCommInitRootInfo")
        else:
            _check(lib.HcclCommInitRootInfoConfig(world_size, byref(info), rank, byref(config), byref(h)), "HcclCommInitRootInfoConfig")
        return cls(h.value, "device")

    @classmethod
    def from_torch_distributed(cls, group=None, config: Optional[_lib.HcclCommConfig] = None):
        """Rendezvous through an initialised ``torch.distributed`` group: rank 0
        creates the root info and broadcasts it (any backend)."""
        import torch.distributed as dist

        rank, world = dist.get_rank(group), dist.get_world_size(group)
        obj = [cls.get_root_info() if rank == 0 else None]
        dist.broadcast_object_list(obj, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        return cls.from_root_info(obj[0], rank, world, config)

    @classmethod
    def from_rank_table(cls, table: str, rank: int, config: Optional[_lib.HcclCommConfig] = None):
        h = c_void_p()
        if config is None:
            _check(lib.HcclCommInitClusterInfo(table.encode(), rank, byref(h)), "HcclCommInitClusterInfo")
        else:
            _check(lib.HcclCommInitClusterInfoConfig(table.encode(), rank, byref(config), byref(h)), "HcclCommInitClusterInfoConfig")
        return cls(h.value, "device")

    @classmethod
    def emulated(cls, n: int, config: Optional[_lib.HcclCommConfig] = None) -> List["Communicator"]:
        hs = (c_void_p * n)()
        _check(lib.HcclCommInitEmulated(n, byref(config) if config is not None else None, hs), "HcclCommInitEmulated")
        return [cls(hs[i], "emulated") for i in range(n)]

    @classmethod
    def host_sim(cls, n: int, topo: Optional[str] = None, config: Optional[_lib.HcclCommConfig] = None) -> List["Communicator"]:
        hs = (c_void_p * n)()
        _check(lib.HcclCommInitHostSim(n, topo.encode() if topo else None, byref(config) if config is not None else None, hs),
               "HcclCommInitHostSim")
        return [cls(hs[i], "host") for i in range(n)]

    def destroy(self) -> None:
        if self._h:
            lib.HcclCommDestroy(self._h)
            self._h = None

    # ------------------------------------------------------------------ queries
    @property
    def handle(self) -> c_void_p:
        return self._h

    @property
    def name(self) -> str:
        buf = ctypes.create_string_buffer(128)
        _check(lib.HcclGetCommName(self._h, buf), "HcclGetCommName")
        return buf.value.decode()

    def status(self) -> CommStatus:
        s = c_int()
        _check(lib.HcclCommGetStatus(self._h, byref(s)), "HcclCommGetStatus")
        return CommStatus(s.value)

    def async_error(self) -> Result:
        e = c_int()
        _check(lib.HcclCommGetAsyncError(self._h, byref(e)), "HcclCommGetAsyncError")
        return Result(e.value)

    def suspend(self) -> None:
        _check(lib.HcclCommSuspend(self._h), "HcclCommSuspend")

    def resume(self) -> None:
        _check(lib.HcclCommResume(self._h), "HcclCommResume")

    def last_algorithm(self) -> str:
        buf = ctypes.create_string_buffer(128)
        _check(lib.HcclGetLastAlgName(self._h, buf, 128), "HcclGetLastAlgName")
        return buf.value.decode()

    def explain(self, op: Cmd, count: int, dtype: DataType, reduce_op: ReduceOp = ReduceOp.SUM, registered: bool = False) -> str:
        buf = ctypes.create_string_buffer(16384)
        lib.HcclSelectorExplain(self._h, int(op), count, int(dtype), int(reduce_op), int(registered), buf, 16384)
        return buf.value.decode()

    def plan_cache_stats(self):
        h, m, n = c_uint64(), c_uint64(), c_uint64()
        _check(lib.HcclGetPlanCacheStats(self._h, byref(h), byref(m), byref(n)), "HcclGetPlanCacheStats")
        return h.value, m.value, n.value

    # ------------------------------------------------------------------ memory
    def empty(self, shape, dtype):
        """A tensor in symmetric memory: collective, same shape on every rank.
        Operators read and write such tensors in place on the peers (zero-copy)."""
        import torch

        numel = int(np.prod(shape))
        nbytes = max(16, numel * torch.empty((), dtype=dtype).element_size())
        p = c_void_p()
        _check(lib.HcclMemAlloc(self._h, nbytes, byref(p)), "HcclMemAlloc")
        self._sym.append((p.value, nbytes))
        raw = torch.as_tensor(_CudaBuffer(p.value, nbytes, self), device="cuda")
        return raw[: numel * torch.empty((), dtype=dtype).element_size()].view(dtype).view(*shape)

    def free(self, tensor) -> None:
        _check(lib.HcclMemFree(self._h, c_void_p(tensor.data_ptr())), "HcclMemFree")
        self._sym = [(p, n) for p, n in self._sym if p != tensor.data_ptr()]

    def is_symmetric(self, tensor) -> bool:
        """True when the tensor starts a block returned by :meth:`empty` that has not been freed."""
        return any(p == tensor.data_ptr() for p, _ in self._sym)

    def register(self, tensor) -> None:
        """Collective: registers a tensor the caller allocated itself (same size on every rank) so that operators use it
        in place on the peers instead of staging it.  Later calls must use the same offsets inside it on every rank."""
        _check(lib.HcclCommRegister(self._h, c_void_p(tensor.data_ptr()), tensor.numel() * tensor.element_size()), "HcclCommRegister")

    def deregister(self, tensor) -> None:
        _check(lib.HcclCommDeregister(self._h, c_void_p(tensor.data_ptr())), "HcclCommDeregister")

    def peer_pointer(self, tensor, peer: int) -> int:
        p = c_void_p()
        _check(lib.HcclCommSymWinGet(self._h, c_void_p(tensor.data_ptr()), peer, byref(p)), "HcclCommSymWinGet")
        return p.value

    # ------------------------------------------------------------------ helpers
    def _buf(self, t):
        """-> (pointer, element count, DataType)"""
        if isinstance(t, np.ndarray):
            if not t.flags["C_CONTIGUOUS"]:
                raise ValueError("numpy buffers must be C-contiguous")
            return c_void_p(t.ctypes.data), t.size, numpy_dtype_map()[t.dtype]
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")
        return c_void_p(t.data_ptr()), t.numel(), torch_dtype_map()[t.dtype]

    def _stream(self, stream=None):
        if self.kind == "host":
            return c_void_p(0)
        if stream is not None:
            return c_void_p(stream.cuda_stream)
        import torch

        # the raw handle of the current stream, without building a torch.cuda.Stream object on every call
        return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))

    # ------------------------------------------------------------------ operators
    def all_reduce(self, send, recv=None, op: ReduceOp = ReduceOp.SUM, stream=None):
        recv = send if recv is None else recv
        sp, n, dt = self._buf(send)
        rp, _, _ = self._buf(recv)
        _check(lib.HcclAllReduce(sp, rp, n, int(dt), int(op), self._h, self._stream(stream)), "HcclAllReduce")
        return recv

    def all_reduce_ex(self, send, recv=None, op: ReduceOp = ReduceOp.SUM, scale: float = 1.0, stream=None):
        """``recv = (recv.dtype)(scale * reduce(send))`` in one pass: ``recv`` may have another floating type than
        ``send`` (fp32 / bf16 / fp16 on either side) and ``scale`` is applied to the fp32 accumulator.  ``scale = 1 /
        world_size`` averages."""
        recv = send if recv is None else recv
        sp, n, dt = self._buf(send)
        rp, _, rdt = self._buf(recv)
        _check(lib.HcclAllReduceEx(sp, rp, n, int(dt), int(rdt), int(op), float(scale), self._h, self._stream(stream)), "HcclAllReduceEx")
        return recv

    def reduce_scatter_ex(self, send, recv, op: ReduceOp = ReduceOp.SUM, scale: float = 1.0, stream=None):
        """ReduceScatter with the output cast to ``recv.dtype`` and scaled, in one pass."""
        sp, _, dt = self._buf(send)
        rp, n, rdt = self._buf(recv)
        _check(lib.HcclReduceScatterEx(sp, rp, n, int(dt), int(rdt), int(op), float(scale), self._h, self._stream(stream)), "HcclReduceScatterEx")
        return recv

    def broadcast(self, buf, root: int = 0, stream=None):
        p, n, dt = self._buf(buf)
        _check(lib.HcclBroadcast(p, n, int(dt), root, self._h, self._stream(stream)), "HcclBroadcast")
        return buf

    def reduce(self, send, recv, root: int = 0, op: ReduceOp = ReduceOp.SUM, stream=None):
        sp, n, dt = self._buf(send)
        rp = self._buf(recv)[0] if recv is not None else c_void_p(0)
        _check(lib.HcclReduce(sp, rp, n, int(dt), int(op), root, self._h, self._stream(stream)), "HcclReduce")
        return recv

    def all_gather(self, send, recv, stream=None):
        sp, n, dt = self._buf(send)
        rp, _, _ = self._buf(recv)
        _check(lib.HcclAllGather(sp, rp, n, int(dt), self._h, self._stream(stream)), "HcclAllGather")
        return recv

    def all_gather_v(self, send, recv, recv_counts, recv_displs, stream=None):
        sp, n, dt = self._buf(send)
        rp, _, _ = self._buf(recv)
        _check(lib.HcclAllGatherV(sp, n, rp, _u64_array(recv_counts), _u64_array(recv_displs), int(dt), self._h, self._stream(stream)),
               "HcclAllGatherV")
        return recv

    def reduce_scatter(self, send, recv, op: ReduceOp = ReduceOp.SUM, stream=None):
        sp, _, dt = self._buf(send)
        rp, n, _ = self._buf(recv)
        _check(lib.HcclReduceScatter(sp, rp, n, int(dt), int(op), self._h, self._stream(stream)), "HcclReduceScatter")
        return recv

    def reduce_scatter_v(self, send, recv, send_counts, send_displs, op: ReduceOp = ReduceOp.SUM, stream=None):
        sp, _, dt = self._buf(send)
        rp, n, _ = self._buf(recv)
        _check(lib.HcclReduceScatterV(sp, _u64_array(send_counts), _u64_array(send_displs), rp, n, int(dt), int(op), self._h,
                                      self._stream(stream)), "HcclReduceScatterV")
        return recv

    def scatter(self, send, recv, root: int = 0, stream=None):
        sp = self._buf(send)[0] if send is not None else c_void_p(0)
        rp, n, dt = self._buf(recv)
        _check(lib.HcclScatter(sp, rp, n, int(dt), root, self._h, self._stream(stream)), "HcclScatter")
        return recv

    def all_to_all(self, send, recv, stream=None):
        sp, n, dt = self._buf(send)
        rp, _, rdt = self._buf(recv)
        per = n // self.world_size
        _check(lib.HcclAlltoAll(sp, per, int(dt), rp, per, int(rdt), self._h, self._stream(stream)), "HcclAlltoAll")
        return recv

    def all_to_all_v(self, send, send_counts, send_displs, recv, recv_counts, recv_displs, stream=None):
        sp, _, dt = self._buf(send)
        rp, _, rdt = self._buf(recv)
        _check(lib.HcclAlltoAllV(sp, _u64_array(send_counts), _u64_array(send_displs), int(dt), rp, _u64_array(recv_counts),
                                 _u64_array(recv_displs), int(rdt), self._h, self._stream(stream)), "HcclAlltoAllV")
        return recv

    def all_to_all_vc(self, send, count_matrix, recv, stream=None):
        sp, _, dt = self._buf(send)
        rp, _, rdt = self._buf(recv)
        flat = [int(v) for row in count_matrix for v in row]
        _check(lib.HcclAlltoAllVC(sp, _u64_array(flat), int(dt), rp, int(rdt), self._h, self._stream(stream)), "HcclAlltoAllVC")
        return recv

    def send(self, buf, dst: int, stream=None):
        p, n, dt = self._buf(buf)
        _check(lib.HcclSend(p, n, int(dt), dst, self._h, self._stream(stream)), "HcclSend")

    def recv(self, buf, src: int, stream=None):
        p, n, dt = self._buf(buf)
        _check(lib.HcclRecv(p, n, int(dt), src, self._h, self._stream(stream)), "HcclRecv")
        return buf

    def batch_send_recv(self, items, stream=None):
        """items: sequence of ("send" | "recv", buffer, peer)."""
        arr = (_lib.HcclSendRecvItem * max(1, len(items)))()
        for i, (kind, buf, peer) in enumerate(items):
            p, n, dt = self._buf(buf)
            arr[i].sendRecvType = 0 if kind == "send" else 1
            arr[i].buf = p
            arr[i].count = n
            arr[i].dataType = int(dt)
            arr[i].remoteRank = peer
        _check(lib.HcclBatchSendRecv(arr, len(items), self._h, self._stream(stream)), "HcclBatchSendRecv")

    def barrier(self, stream=None):
        _check(lib.HcclBarrier(self._h, self._stream(stream)), "HcclBarrier")

    # ------------------------------------------------------------------ host trace / verifier
    def trace_begin(self):
        _check(lib.HcclHostTraceBegin(self._h), "HcclHostTraceBegin")

    def trace_verify(self) -> str:
        buf = ctypes.create_string_buffer(65536)
        code = lib.HcclHostTraceVerify(self._h, buf, 65536)
        if code != 0:
            raise HcclError(code, "HcclHostTraceVerify: " + buf.value.decode())
        return buf.value.decode()


def registry():
    """[(name, Cmd, Engine)] of every registered algorithm."""
    out = []
    for i in range(lib.HcclAlgRegistryCount()):
        buf = ctypes.create_string_buffer(128)
        op, eng = c_int(), c_int()
        _check(lib.HcclAlgRegistryEntry(i, buf, 128, byref(op), byref(eng)), "HcclAlgRegistryEntry")
        out.append((buf.value.decode(), op.value, eng.value))
    return out
