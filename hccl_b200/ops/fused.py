"""Single-pass bf16 kernels for the memory-bound pieces of a decoder layer, with autograd:

* ``add_rms_norm(x, delta, weight, eps)`` -> ``(x + delta, rms_norm(x + delta) * weight)`` (``delta=None``: norm only)
* ``swiglu(gate_up)`` -> ``silu(gate) * up`` for ``gate_up = [gate | up]`` along the last dimension
* ``rope(x, cos, sin)`` -> rotary embedding ("rotate halves") of ``x [S, heads, D]``; ``x`` may be a column slice
  of a wider projection output (row stride larger than ``heads * D``)

CUDA bf16 tensors run the hand-written kernels (csrc/kernels/fused_elementwise.cu); anything else (CPU tensors, other
dtypes, hidden > 8192) takes the equivalent PyTorch expression, which is also the reference the tests compare against.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from .._lib import lib
from ..comm import _check


LAUNCHES = 0          # kernels of this module launched so far (benchmark accounting)


def _count(n=1):
    global LAUNCHES
    LAUNCHES += n


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _s():
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _native(*tensors, hidden=None) -> bool:
    for t in tensors:
        if t is None:
            continue
        if not (t.is_cuda and t.dtype == torch.bfloat16):
            return False
    if hidden is not None and (hidden % 8 != 0 or hidden > 8192):
        return False
    if not hasattr(lib, "HcclFusedRope"):
        raise RuntimeError("libhccl_b200.so predates the fused element-wise kernels: rebuild it with `python hccl_b200/build.py`")
    return True


# ----------------------------------------------------------------------------- reference expressions
def add_rms_norm_reference(x, delta, weight, eps):
    x_out = x if delta is None else x + delta
    return x_out, F.rms_norm(x_out, (x_out.shape[-1],), weight, eps)


def swiglu_reference(gate_up):
    g, u = gate_up.chunk(2, dim=-1)
    return F.silu(g) * u


def rope_reference(x, cos, sin):
    d = x.shape[-1] // 2
    x1, x2 = x[..., :d].float(), x[..., d:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1).to(x.dtype)


# ----------------------------------------------------------------------------- autograd functions
class _AddRmsNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, delta, weight, eps):
        rows, hidden = x.numel() // x.shape[-1], x.shape[-1]
        x = x.contiguous()
        h = torch.empty_like(x)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        if delta is not None:
            delta = delta.contiguous()
            x_out = torch.empty_like(x)
        else:
            x_out = x
        _check(lib.HcclFusedAddRmsNormFwd(_p(x), _p(delta), _p(weight), _p(x_out) if delta is not None else ctypes.c_void_p(0), _p(h), _p(rstd),
                                          rows, hidden, float(eps), _s()), "HcclFusedAddRmsNormFwd")
        _count()
        ctx.save_for_backward(x_out, weight, rstd)
        ctx.has_delta = delta is not None
        return (x_out, h) if delta is not None else h        # without delta the input itself is the residual stream

    @staticmethod
    def backward(ctx, *grads):
        dx_out, dh = grads if ctx.has_delta else (None, grads[0])
        x_out, weight, rstd = ctx.saved_tensors
        rows, hidden = x_out.numel() // x_out.shape[-1], x_out.shape[-1]
        if dh is None:
            dh = torch.zeros_like(x_out)
        dh = dh.contiguous()
        extra = dx_out.contiguous() if dx_out is not None else None
        dx = torch.empty_like(x_out)
        dw = torch.empty_like(weight)
        n_part = lib.HcclFusedRmsNormBwdPartials(rows)
        partial = torch.empty((n_part, hidden), device=x_out.device, dtype=torch.float32)
        _check(lib.HcclFusedRmsNormBwd(_p(dh), _p(x_out), _p(weight), _p(rstd), _p(extra), _p(dx), _p(partial), _p(dw), rows, hidden, _s()),
               "HcclFusedRmsNormBwd")
        _count(2)
        return dx, (dx if ctx.has_delta else None), dw, None


class _Swiglu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        gate_up = gate_up.contiguous()
        f = gate_up.shape[-1] // 2
        rows = gate_up.numel() // gate_up.shape[-1]
        out = torch.empty(gate_up.shape[:-1] + (f,), device=gate_up.device, dtype=gate_up.dtype)
        _check(lib.HcclFusedSwigluFwd(_p(gate_up), _p(out), rows, f, _s()), "HcclFusedSwigluFwd")
        _count()
        ctx.save_for_backward(gate_up)
        return out

    @staticmethod
    def backward(ctx, dout):
        (gate_up,) = ctx.saved_tensors
        f = gate_up.shape[-1] // 2
        rows = gate_up.numel() // gate_up.shape[-1]
        dgu = torch.empty_like(gate_up)
        _check(lib.HcclFusedSwigluBwd(_p(gate_up), _p(dout.contiguous()), _p(dgu), rows, f, _s()), "HcclFusedSwigluBwd")
        _count()
        return dgu


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        s, nh, d = x.shape
        assert x.stride(2) == 1 and x.stride(1) == d, "rope: heads must be packed inside a row"
        out = torch.empty((s, nh, d), device=x.device, dtype=x.dtype)
        _check(lib.HcclFusedRope(_p(x), x.stride(0), _p(out), nh * d, _p(cos), _p(sin), s, nh, d, 0, _s()), "HcclFusedRope")
        _count()
        ctx.save_for_backward(cos, sin)
        return out

    @staticmethod
    def backward(ctx, dout):
        cos, sin = ctx.saved_tensors
        s, nh, d = dout.shape
        dout = dout.contiguous()
        dx = torch.empty_like(dout)
        _check(lib.HcclFusedRope(_p(dout), nh * d, _p(dx), nh * d, _p(cos), _p(sin), s, nh, d, 1, _s()), "HcclFusedRope")
        _count()
        return dx, None, None


# ----------------------------------------------------------------------------- public functions
def add_rms_norm(x, delta, weight, eps: float = 1e-5, use_kernels: bool = True):
    """``x_out = x + delta`` (``delta`` may be None) and ``h = rms_norm(x_out) * weight`` in one pass; returns both."""
    if use_kernels and _native(x, delta, weight, hidden=x.shape[-1]):
        if delta is None:
            return x, _AddRmsNorm.apply(x, None, weight, eps)
        return _AddRmsNorm.apply(x, delta, weight, eps)
    return add_rms_norm_reference(x, delta, weight, eps)


def swiglu(gate_up, use_kernels: bool = True):
    if use_kernels and _native(gate_up) and (gate_up.shape[-1] // 2) % 8 == 0:
        return _Swiglu.apply(gate_up)
    return swiglu_reference(gate_up)


def rope(x, cos, sin, use_kernels: bool = True):
    """x [S, heads, D] (row stride may exceed heads * D), cos / sin fp32 [S, D / 2]."""
    if (use_kernels and _native(x) and x.shape[-1] % 16 == 0 and x.stride(2) == 1 and x.stride(1) == x.shape[-1] and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and cos.dtype == torch.float32 and cos.is_contiguous() and sin.is_contiguous()):
        return _Rope.apply(x, cos, sin)
    return rope_reference(x, cos, sin)
