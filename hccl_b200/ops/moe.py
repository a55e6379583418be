"""Expert-parallel MoE dispatch / combine on the fused kernels.

``MoeDispatcher`` owns the symmetric receive buffers of one expert-parallel
group.  ``dispatch`` sends every (token, expert) pair to the rank that hosts the
expert - the row is quantised to fp8 e4m3 with one fp32 scale per 1x128 block
on the way - and returns the received rows grouped by local expert.  ``combine``
pulls the expert outputs back and applies the gate weights in the same pass.
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from .. import _lib
from .._lib import lib
from ..comm import Communicator, _check


@dataclasses.dataclass
class DispatchResult:
    x_fp8: torch.Tensor         # [capacity, hidden] float8_e4m3fn (rows beyond offsets[-1] are unused)
    scales: torch.Tensor        # [capacity, hidden // 128] fp32
    src_info: torch.Tensor      # [capacity] int64: (source rank << 32) | (token * topk + k)
    offsets: torch.Tensor       # [experts_per_rank + 1] int32 row ranges per local expert
    slot_map: torch.Tensor      # [tokens * topk] int64, input of combine


class MoeDispatcher:
    def __init__(self, comm: Communicator, n_tokens: int, hidden: int, topk: int, n_experts: int, capacity: int | None = None):
        self.comm = comm
        self.cfg = _lib.HcclMoeConfig(n_tokens, hidden, topk, n_experts, capacity or 2 * n_tokens * topk)
        cap = self.cfg.capacity
        self.recv_x = comm.empty((cap, hidden), torch.uint8)
        self.recv_scale = comm.empty((cap, hidden // 128), torch.float32)
        self.recv_src = comm.empty((cap,), torch.int64)
        self.y = comm.empty((cap, hidden), torch.bfloat16)          # expert outputs, read by the peers in combine
        self.offsets = torch.zeros(n_experts // comm.world_size + 1, dtype=torch.int32, device="cuda")
        self.slot_map = torch.zeros(n_tokens * topk, dtype=torch.int64, device="cuda")

    def _stream(self, stream=None):
        s = stream if stream is not None else torch.cuda.current_stream()
        return ctypes.c_void_p(s.cuda_stream)

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, stream=None) -> DispatchResult:
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        _check(lib.HcclMoeDispatch(self.comm.handle, p(x), p(topk_idx), ctypes.byref(self.cfg), p(self.recv_x), p(self.recv_scale), p(self.recv_src),
                                   p(self.offsets), p(self.slot_map), self._stream(stream)), "HcclMoeDispatch")
        return DispatchResult(self.recv_x.view(torch.float8_e4m3fn), self.recv_scale, self.recv_src, self.offsets, self.slot_map)

    def combine(self, topk_weight: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
        """``out[t] = sum_k topk_weight[t, k] * y[slot(t, k)]`` with ``self.y`` holding the expert outputs."""
        assert topk_weight.dtype == torch.float32 and topk_weight.is_contiguous()
        if out is None:
            out = torch.empty((self.cfg.nTokens, self.cfg.hidden), dtype=torch.bfloat16, device="cuda")
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        _check(lib.HcclMoeCombine(self.comm.handle, p(self.y), p(topk_weight), p(self.slot_map), ctypes.byref(self.cfg), p(out), self._stream(stream)),
               "HcclMoeCombine")
        return out


def dequantize(x_fp8: torch.Tensor, scales: torch.Tensor) -> torch.Tensor:
    """Reference dequantisation of block-scaled rows: [rows, hidden] fp8 x [rows, hidden / 128] -> fp32."""
    rows, hidden = x_fp8.shape
    return (x_fp8.float().view(rows, hidden // 128, 128) * scales.view(rows, hidden // 128, 1)).view(rows, hidden)


def expert_offsets(topk_idx: torch.Tensor, n_experts: int, stream=None) -> torch.Tensor:
    """Row range of every expert when this rank's (token, expert) pairs are grouped by expert: int32 [n_experts + 1]."""
    assert topk_idx.dtype == torch.int32 and topk_idx.is_contiguous()
    out = torch.empty(n_experts + 1, dtype=torch.int32, device=topk_idx.device)
    s = stream if stream is not None else torch.cuda.current_stream()
    _check(lib.HcclMoeExpertOffsets(ctypes.c_void_p(topk_idx.data_ptr()), topk_idx.numel(), n_experts, ctypes.c_void_p(out.data_ptr()),
                                    ctypes.c_void_p(s.cuda_stream)), "HcclMoeExpertOffsets")
    return out
