"""Data-parallel gradient synchronisation on the AllReduce operator.

The reference provides the collectives data parallelism consumes (AllReduce for replicated gradients, ReduceScatter +
AllGather for sharded ones, docs/en/architecture-brief.md:16-17) and leaves the bucketing to the framework.  This is
that thin framework side for plain PyTorch modules:

* gradients are packed into flat buckets of about ``bucket_mib`` MiB, in reverse parameter order (the order in which
  backward produces them);
* ``overlap=True`` hooks every parameter: when the last gradient of a bucket has been accumulated, the bucket's
  AllReduce is issued at once - on a side stream for CUDA tensors, so that it runs beside the rest of backward - and
  buckets are always issued in index order, which keeps the ranks' call sequences identical;
* the average is part of the AllReduce (``all_reduce_ex`` with ``scale = 1 / world``: the kernel scales its fp32
  accumulator before it stores), so no separate pass divides the bucket;
* on a device communicator the flat buckets live in symmetric memory (``comm.empty``), which the kernels read and
  write in place on the peers instead of staging them through the slab;
* ``finish()`` (or ``reduce()`` without hooks) waits for the side stream and writes the reduced values back into
  ``p.grad``.

NVSwitch gives every GPU full bandwidth to every peer, so a bucket is sized for launch latency and overlap (tens of
MiB), not for link count.
"""
from __future__ import annotations

from typing import Iterable, List

import torch


class GradientBucketer:
    def __init__(self, params: Iterable[torch.nn.Parameter], comm, bucket_mib: float = 25.0, average: bool = True, overlap: bool = False):
        self.comm = comm
        self.average = average
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        order = list(reversed(self.params))
        limit = int(bucket_mib * (1 << 20))
        self.buckets: List[List[torch.nn.Parameter]] = []
        cur, cur_bytes, cur_key = [], 0, None
        for p in order:
            key = (p.dtype, p.device)
            nbytes = p.numel() * p.element_size()
            if cur and (key != cur_key or cur_bytes + nbytes > limit):
                self.buckets.append(cur)
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_key = key
        if cur:
            self.buckets.append(cur)
        self._float_types = (torch.float32, torch.bfloat16, torch.float16)
        self.flat = []
        for b in self.buckets:
            numel = sum(p.numel() for p in b)
            if b[0].is_cuda and getattr(comm, "kind", "") == "device" and comm.world_size > 1:
                buf = comm.empty((numel,), b[0].dtype)          # collective: every rank builds the same buckets in the same order
                buf.zero_()
            else:
                buf = torch.zeros(numel, dtype=b[0].dtype, device=b[0].device)
            self.flat.append(buf)
        self._bucket_of = {p: i for i, b in enumerate(self.buckets) for p in b}
        self._pending = [0] * len(self.buckets)
        self._next = 0
        self._launched = [False] * len(self.buckets)
        self._stream = None
        self._hooks = []
        if overlap:
            for p in self.params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))
        self._reset()

    # ------------------------------------------------------------------ internals
    def _reset(self):
        self._pending = [len(b) for b in self.buckets]
        self._launched = [False] * len(self.buckets)
        self._next = 0

    def _side_stream(self, device):
        if device.type != "cuda":
            return None
        if self._stream is None:
            self._stream = torch.cuda.Stream(device=device)
        return self._stream

    def _launch(self, i: int):
        bucket, flat = self.buckets[i], self.flat[i]
        side = self._side_stream(flat.device)
        if side is not None:
            side.wait_stream(torch.cuda.current_stream(flat.device))      # the gradients of this bucket are complete
        ctx = torch.cuda.stream(side) if side is not None else _Null()
        with ctx:
            off = 0
            for p in bucket:
                n = p.numel()
                if p.grad is None:
                    flat[off:off + n].zero_()          # a parameter that took no part in this step contributes zeros
                else:
                    flat[off:off + n].copy_(p.grad.reshape(-1))
                off += n
            fused = self.average and flat.dtype in self._float_types and self.comm.world_size > 1
            scale = 1.0 / self.comm.world_size if fused else 1.0
            kw = {"stream": side} if side is not None else {}
            if fused:
                self.comm.all_reduce_ex(flat, flat, scale=scale, **kw)
            else:
                self.comm.all_reduce(flat, flat, **kw)
        self._launched[i] = True

    def _on_grad(self, p):
        i = self._bucket_of[p]
        self._pending[i] -= 1
        # issue every bucket that is complete, in index order only
        while self._next < len(self.buckets) and self._pending[self._next] == 0:
            self._launch(self._next)
            self._next += 1

    # ------------------------------------------------------------------ API
    def reduce(self):
        """Synchronises every gradient now (no hooks needed)."""
        for i in range(len(self.buckets)):
            if not self._launched[i]:
                self._launch(i)
        self.finish()

    def finish(self):
        """Waits for the issued buckets (launching those whose parameters never produced a gradient), then writes the
        reduced gradients back."""
        for i in range(len(self.buckets)):
            if not self._launched[i]:
                self._launch(i)
        if self._stream is not None:
            torch.cuda.current_stream(self._stream.device).wait_stream(self._stream)
        for bucket, flat in zip(self.buckets, self.flat):
            if self.average and flat.dtype not in self._float_types:
                flat.div_(self.comm.world_size, rounding_mode="floor") if not flat.dtype.is_floating_point else flat.mul_(1.0 / self.comm.world_size)
            off = 0
            for p in bucket:
                n = p.numel()
                if p.grad is None:
                    p.grad = flat[off:off + n].reshape(p.shape).clone()
                else:
                    p.grad.copy_(flat[off:off + n].reshape(p.shape))
                off += n
        self._reset()

    def remove_hooks(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []


class _Null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


class ShardedOptimizer:
    """Sharded data parallelism on ReduceScatter + AllGather (the second DP form the reference's documents name,
    docs/en/architecture-brief.md:16-17): every rank keeps the optimizer state of 1 / P of the parameters.

    ``step()``: the gradients are packed into one flat buffer, ReduceScatter leaves every rank with the sum of its
    shard, the inner optimizer (built by ``optimizer_factory`` over ONE flat shard parameter) updates that shard, and
    AllGather hands every rank the updated parameters.  All parameters must share dtype and device.  The flat buffer
    is padded to a multiple of the world size; the padding is never read back.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], comm, optimizer_factory, average: bool = True):
        self.comm = comm
        self.average = average
        self.params = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("ShardedOptimizer: no trainable parameters")
        dt, dev = self.params[0].dtype, self.params[0].device
        if any(p.dtype != dt or p.device != dev for p in self.params):
            raise ValueError("ShardedOptimizer: parameters must share dtype and device")
        P = comm.world_size
        total = sum(p.numel() for p in self.params)
        self.shard_len = (total + P - 1) // P
        self.flat_grad = torch.zeros(self.shard_len * P, dtype=dt, device=dev)
        self.flat_param = torch.zeros(self.shard_len * P, dtype=dt, device=dev)
        self._pack(self.flat_param, [p.detach() for p in self.params])
        r = comm.rank
        self.shard = torch.nn.Parameter(self.flat_param[r * self.shard_len:(r + 1) * self.shard_len].clone())
        self.shard.grad = torch.zeros_like(self.shard)
        self.optimizer = optimizer_factory([self.shard])

    def _pack(self, flat, tensors):
        off = 0
        for t in tensors:
            n = t.numel()
            flat[off:off + n].copy_(t.reshape(-1))
            off += n

    @torch.no_grad()
    def step(self):
        off = 0
        for p in self.params:
            n = p.numel()
            if p.grad is None:
                self.flat_grad[off:off + n].zero_()
            else:
                self.flat_grad[off:off + n].copy_(p.grad.reshape(-1))
            off += n
        if self.average and self.flat_grad.dtype in (torch.float32, torch.bfloat16, torch.float16) and self.comm.world_size > 1:
            self.comm.reduce_scatter_ex(self.flat_grad, self.shard.grad, scale=1.0 / self.comm.world_size)      # averaged in the same pass
        else:
            self.comm.reduce_scatter(self.flat_grad, self.shard.grad)
            if self.average:
                self.shard.grad.mul_(1.0 / self.comm.world_size)
        self.optimizer.step()
        self.comm.all_gather(self.shard.detach(), self.flat_param)
        off = 0
        for p in self.params:
            n = p.numel()
            p.copy_(self.flat_param[off:off + n].reshape(p.shape))
            off += n

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
