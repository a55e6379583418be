"""Tensor-parallel + sequence-parallel linear layers on the MC2 fused kernels.

Megatron-style sequence parallelism: activations between blocks are sharded over
the sequence dimension; a column-parallel linear starts with an all-gather of
the sequence shards and a row-parallel linear ends with a reduce-scatter.  Both
are ONE kernel here (tcgen05 matmul + collective), forward and backward:

  column-parallel   y = all_gather(x) @ W^T            forward : AllGather->Matmul
                    dx = reduce_scatter(dy @ W)        backward: Matmul->ReduceScatter
                    dW = dy^T @ all_gather(x)                    plain matmul (gathered x saved by the forward)
  row-parallel      y = reduce_scatter(x @ W^T)        forward : Matmul->ReduceScatter
                    dx = all_gather(dy) @ W            backward: AllGather->Matmul
                    dW = all_gather(dy)^T @ x                    plain matmul (gathered dy from the backward kernel)

With ``impl="nccl"`` the same layers run on torch.distributed (NCCL) collectives
and torch.matmul (cuBLAS): the comparison baseline.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..ops import mc2


class TPContext:
    """What the layers need to know about the tensor-parallel group."""

    def __init__(self, comm=None, group=None, impl: str = "hccl", device="cuda", dtype=torch.bfloat16, fused_ops=None):
        self.comm = comm                  # hccl_b200.Communicator (impl == "hccl")
        self.group = group                # torch.distributed group (impl == "nccl"; any backend, gloo on CPU included)
        self.impl = impl
        self.device = device              # where parameters and activations live ("cpu" only with impl == "nccl")
        self.dtype = dtype
        if impl == "hccl":
            self.world = comm.world_size if comm is not None else 1
            self.rank = comm.rank if comm is not None else 0
        else:
            self.world = dist.get_world_size(group) if dist.is_initialized() else 1
            self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._sym = {}
        self.launches = 0                 # kernels of this library launched (bench accounting)
        # AllGather->Matmul form: "push" (every rank writes its shard into the others' symmetric gathered buffers) or
        # "pull" (every rank reads the peers' symmetric shards)
        import os
        # measured: push wins at 2 ranks (0.38 vs 0.40 ms), pull at 8 (0.43 vs 0.47 ms with 28 workers)
        self.ag_form = os.environ.get("HCCL_TP_AG_FORM", "push" if self.world <= 2 else "pull")
        # residual add + RMSNorm, SwiGLU and rotary embedding as this library's single-pass kernels (the NCCL + cuBLAS
        # comparison arm keeps the framework's element-wise kernels); HCCL_FUSED_ELEMENTWISE=0 turns them off
        # ``fused_ops=True`` also gives them to the NCCL + cuBLAS arm, so that the two arms differ in the collectives
        # and the matmul kernels only
        if fused_ops is None:
            fused_ops = impl == "hccl"
        self.fused_ops = bool(fused_ops) and str(device).startswith("cuda") and os.environ.get("HCCL_FUSED_ELEMENTWISE", "1") != "0"

    # ---- collectives on whole tensors, either arm (used for what is not a fused matmul: the embedding exchange and
    # the gradients of replicated parameters)
    def all_to_all(self, send, key):
        """``send [P, ...]``: block q goes to rank q; returns ``[P, ...]`` whose block q came from rank q."""
        if self.world == 1:
            return send
        if self.impl == "hccl":
            buf = self.sym_buffer(("a2a_send", key), send.shape, send.dtype)
            buf.copy_(send)
            recv = torch.empty_like(send)
            self.comm.all_to_all(buf, recv)
            self.launches += 1
            return recv
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send.contiguous(), group=self.group)
        return recv

    def all_reduce_(self, t, key):
        """In-place sum over the group."""
        if self.world == 1:
            return t
        if self.impl == "hccl":
            self.comm.all_reduce(t)
            self.launches += 1
        else:
            dist.all_reduce(t, group=self.group)
        return t

    def flat_buffer(self, key, numel, dtype):
        """A flat scratch tensor that the all-reduce of this arm takes at full speed (symmetric memory for the library)."""
        if self.impl == "hccl" and self.world > 1:
            return self.sym_buffer(("flat", key), (numel,), dtype)
        k = ("flat", key, numel, dtype)
        buf = self._sym.get(k)
        if buf is None:
            buf = torch.empty(numel, device=self.device, dtype=dtype)
            self._sym[k] = buf
        return buf

    def release(self):
        """Frees the symmetric buffers of this context (collective: every rank calls it)."""
        bufs, self._sym = self._sym, {}
        if self.impl == "hccl" and self.comm is not None:
            torch.cuda.synchronize()
            for k in sorted(bufs, key=repr):              # same order on every rank
                if bufs[k].is_cuda and self.comm.is_symmetric(bufs[k]):
                    self.comm.free(bufs[k])

    def sym_buffer(self, key, shape, dtype=torch.bfloat16):
        """A persistent symmetric buffer per call site and shape (allocated collectively on first use)."""
        k = (key, tuple(shape), dtype)
        buf = self._sym.get(k)
        if buf is None:
            buf = self.comm.empty(tuple(shape), dtype)
            self._sym[k] = buf
        return buf


def _reduce_scatter_rows(ctx, full):
    """Framework arm: ``[S, N] -> [S / P, N]`` summed over the group (backends without a reduce-scatter, gloo on CPU,
    take an all-reduce and keep their rows)."""
    rows = full.shape[0] // ctx.world
    out = torch.empty((rows, full.shape[1]), device=full.device, dtype=full.dtype)
    if full.is_cuda:
        dist.reduce_scatter_tensor(out, full, group=ctx.group)
    else:
        full = full.clone()
        dist.all_reduce(full, group=ctx.group)
        out.copy_(full[ctx.rank * rows:(ctx.rank + 1) * rows])
    return out


def _mm(ctx, a, b, **kw):
    if ctx.impl == "hccl":
        ctx.launches += 1
        return mc2.matmul(a, b, **kw)
    A = a.t() if kw.get("trans_a", False) else a
    B = b.t() if kw.get("trans_b", True) else b
    return A @ B


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(fctx, x_shard, weight, ctx: TPContext, key):
        # x_shard [S/P, K], weight [N_local, K]
        if ctx.world == 1:
            fctx.save_for_backward(x_shard, weight)
            fctx.ctx, fctx.key = ctx, key
            return _mm(ctx, x_shard, weight)
        if ctx.impl == "hccl":
            # push form: the gathered activations land in a persistent symmetric buffer of this call site (every rank
            # writes its shard into the others' buffers); the shard itself is read where it is
            if ctx.ag_form == "push":
                gathered = ctx.sym_buffer(("cp_gathered", key), (x_shard.shape[0] * ctx.world, x_shard.shape[1]))
                out, gathered = mc2.all_gather_matmul(ctx.comm, x_shard.contiguous(), weight, gathered=gathered)
            else:
                a = ctx.sym_buffer(("cp_in", key), x_shard.shape)
                a.copy_(x_shard)
                out, gathered = mc2.all_gather_matmul(ctx.comm, a, weight)
            ctx.launches += 1
        else:
            gathered = torch.empty((x_shard.shape[0] * ctx.world, x_shard.shape[1]), device=x_shard.device, dtype=x_shard.dtype)
            dist.all_gather_into_tensor(gathered, x_shard.contiguous(), group=ctx.group)
            out = gathered @ weight.t()
        fctx.save_for_backward(gathered, weight)
        fctx.ctx, fctx.key = ctx, key
        return out

    @staticmethod
    def backward(fctx, dy):
        x_full, weight = fctx.saved_tensors
        ctx = fctx.ctx
        dy = dy.contiguous()
        dw = _mm(ctx, dy, x_full, trans_a=True, trans_b=False)           # [N_local, K]
        if ctx.world == 1:
            dx = _mm(ctx, dy, weight, trans_b=False)
        elif ctx.impl == "hccl":
            dx = mc2.matmul_reduce_scatter(ctx.comm, dy, weight, weight_is_kn=True)
            ctx.launches += 1
        else:
            dx = _reduce_scatter_rows(ctx, dy @ weight)
        return dx, dw, None, None


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(fctx, x, weight, ctx: TPContext, key):
        # x [S, K_local], weight [N, K_local]
        fctx.save_for_backward(x, weight)
        fctx.ctx, fctx.key = ctx, key
        if ctx.world == 1:
            return _mm(ctx, x, weight)
        if ctx.impl == "hccl":
            ctx.launches += 1
            return mc2.matmul_reduce_scatter(ctx.comm, x.contiguous(), weight)
        return _reduce_scatter_rows(ctx, x @ weight.t())

    @staticmethod
    def backward(fctx, dy_shard):
        x, weight = fctx.saved_tensors
        ctx = fctx.ctx
        dy_shard = dy_shard.contiguous()
        if ctx.world == 1:
            dx = _mm(ctx, dy_shard, weight, trans_b=False)
            dw = _mm(ctx, dy_shard, x, trans_a=True, trans_b=False)
            return dx, dw, None, None
        if ctx.impl == "hccl":
            if ctx.ag_form == "push":
                dy_full = ctx.sym_buffer(("rp_dy_gathered", dy_shard.shape[1]), (dy_shard.shape[0] * ctx.world, dy_shard.shape[1]))
                dx, dy_full = mc2.all_gather_matmul(ctx.comm, dy_shard, weight, weight_is_kn=True, gathered=dy_full)
            else:
                a = ctx.sym_buffer(("rp_dy", fctx.key), dy_shard.shape)
                a.copy_(dy_shard)
                dx, dy_full = mc2.all_gather_matmul(ctx.comm, a, weight, weight_is_kn=True)
            ctx.launches += 1
        else:
            dy_full = torch.empty((dy_shard.shape[0] * ctx.world, dy_shard.shape[1]), device=dy_shard.device, dtype=dy_shard.dtype)
            dist.all_gather_into_tensor(dy_full, dy_shard, group=ctx.group)
            dx = dy_full @ weight
        dw = _mm(ctx, dy_full, x, trans_a=True, trans_b=False)           # [N, K_local]
        return dx, dw, None, None


class ColumnParallelLinear(torch.nn.Module):
    """``y[S, N/P] = all_gather(x[S/P, K]) @ W^T`` with the weight sharded over its rows (output features)."""

    shard_dim = 0             # the full weight [out, in] is cut along this dimension

    def __init__(self, in_features, out_features, ctx: TPContext, key, std=0.02):
        super().__init__()
        assert out_features % ctx.world == 0
        self.ctx, self.key = ctx, key
        self.weight = torch.nn.Parameter(torch.randn(out_features // ctx.world, in_features, device=ctx.device, dtype=torch.float32).mul_(std).to(ctx.dtype))

    def forward(self, x_shard):
        return _ColumnParallel.apply(x_shard, self.weight, self.ctx, self.key)


class RowParallelLinear(torch.nn.Module):
    """``y[S/P, N] = reduce_scatter(x[S, K/P] @ W^T)`` with the weight sharded over its columns (input features)."""

    shard_dim = 1

    def __init__(self, in_features, out_features, ctx: TPContext, key, std=0.02):
        super().__init__()
        assert in_features % ctx.world == 0
        self.ctx, self.key = ctx, key
        self.weight = torch.nn.Parameter(torch.randn(out_features, in_features // ctx.world, device=ctx.device, dtype=torch.float32).mul_(std).to(ctx.dtype))

    def forward(self, x):
        return _RowParallel.apply(x, self.weight, self.ctx, self.key)
