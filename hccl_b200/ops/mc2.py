"""MC2: matmul fused with a collective, and the plain tcgen05 matmul they share.

All operands are bf16 CUDA tensors; accumulation is fp32.  ``weight`` follows the
``torch.nn.Linear`` convention ``[out_features, in_features]`` unless
``weight_is_kn`` says the matrix is stored ``[K, N]``.
"""
from __future__ import annotations

import ctypes

import torch

from .._lib import lib
from ..comm import Communicator, _check


def _s(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def matmul(a: torch.Tensor, b: torch.Tensor, *, trans_a: bool = False, trans_b: bool = True, out: torch.Tensor | None = None, stream=None):
    """``out[M, N] = op(a) @ op(b)``.

    ``trans_a=False``: ``a`` is ``[M, K]``; ``True``: ``a`` is ``[K, M]``.
    ``trans_b=True``: ``b`` is ``[N, K]`` (a Linear weight); ``False``: ``b`` is ``[K, N]``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and a.is_contiguous() and b.is_contiguous()
    m, k = (a.shape[1], a.shape[0]) if trans_a else (a.shape[0], a.shape[1])
    n = b.shape[0] if trans_b else b.shape[1]
    kb = b.shape[1] if trans_b else b.shape[0]
    assert k == kb, f"inner dimensions differ: {k} vs {kb}"
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    _check(lib.HcclMc2Matmul(_p(a), _p(b), _p(out), m, n, k, int(trans_a), int(trans_b), _s(stream)), "HcclMc2Matmul")
    return out


def all_gather_matmul(comm: Communicator, a_shard: torch.Tensor, weight: torch.Tensor, *, weight_is_kn: bool = False,
                      out: torch.Tensor | None = None, gathered: torch.Tensor | None = None, stream=None):
    """``out = all_gather(a_shard, dim=0) @ W``.  Returns ``(out, gathered)`` - the gathered activations are a
    by-product the backward pass reuses.

    Two forms.  Push (faster: posted writes over NVLink): pass ``gathered`` allocated with ``comm.empty``; every rank
    stores its shard into all ranks' gathered buffers and ``a_shard`` may be any tensor.  Pull: ``a_shard`` is
    symmetric memory and ``gathered`` a plain (or omitted) tensor; every rank reads the peers' shards."""
    m_per, k = a_shard.shape
    n = weight.shape[1] if weight_is_kn else weight.shape[0]
    p = comm.world_size
    if out is None:
        out = torch.empty((m_per * p, n), device=a_shard.device, dtype=torch.bfloat16)
    if gathered is None:
        gathered = torch.empty((m_per * p, k), device=a_shard.device, dtype=torch.bfloat16)
    _check(lib.HcclMc2AllGatherMatmul(_p(a_shard), _p(weight), _p(out), _p(gathered), m_per, n, k, int(not weight_is_kn), comm.handle,
                                      _s(stream)), "HcclMc2AllGatherMatmul")
    return out, gathered


def matmul_reduce_scatter(comm: Communicator, a: torch.Tensor, weight: torch.Tensor, *, weight_is_kn: bool = False,
                          out: torch.Tensor | None = None, stream=None):
    """``out[M / P, N] = reduce_scatter(a @ W, dim=0)``."""
    m, k = a.shape
    n = weight.shape[1] if weight_is_kn else weight.shape[0]
    if out is None:
        out = torch.empty((m // comm.world_size, n), device=a.device, dtype=torch.bfloat16)
    _check(lib.HcclMc2MatmulReduceScatter(_p(a), _p(weight), _p(out), m, n, k, int(not weight_is_kn), comm.handle, _s(stream)),
           "HcclMc2MatmulReduceScatter")
    return out


def matmul_all_reduce(comm: Communicator, a: torch.Tensor, weight: torch.Tensor, *, out: torch.Tensor | None = None, stream=None):
    """``out[M, N] = all_reduce(a @ W^T)`` for decode-sized M (weight ``[N, K]``)."""
    m, k = a.shape
    n = weight.shape[0]
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=torch.bfloat16)
    _check(lib.HcclMc2MatmulAllReduce(_p(a), _p(weight), _p(out), m, n, k, 1, comm.handle, _s(stream)), "HcclMc2MatmulAllReduce")
    return out
