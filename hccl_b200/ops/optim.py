"""AdamW whose update runs as one kernel launch per 80 tensors (csrc/kernels/fused_optimizer.cu).

``FusedAdamW`` follows ``torch.optim.AdamW`` (decoupled weight decay, bias correction, eps outside the square root;
no amsgrad, no maximize).  The moments are kept in the parameters' dtype unless ``state_dtype`` says otherwise
(bf16 parameters with bf16 or fp32 moments, fp32 with fp32).  The step counter lives on the device and the tensor
table travels in the kernel's parameter space, so ``step()`` can be captured in a CUDA graph: moments and counter are
created in the constructor, not on the first step.  CPU parameters and other dtypes take the equivalent PyTorch
expressions, which are also what the tests compare the kernel against.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, Optional

import torch

from .._lib import lib
from ..comm import _check
from ..types import DataType
from . import fused as _fused


class _AdamTensor(ctypes.Structure):
    _fields_ = [("param", ctypes.c_void_p), ("grad", ctypes.c_void_p), ("expAvg", ctypes.c_void_p), ("expAvgSq", ctypes.c_void_p),
                ("numel", ctypes.c_uint64)]


_DT = {torch.bfloat16: DataType.BFP16, torch.float32: DataType.FP32}


def adamw_reference_(p, g, m, v, step: int, lr: float, beta1: float, beta2: float, eps: float, weight_decay: float) -> None:
    """One AdamW update in fp32 math on tensors of any dtype (in place); `step` counts from 1."""
    pf, gf, mf, vf = p.float(), g.float(), m.float(), v.float()
    pf.mul_(1.0 - lr * weight_decay)
    mf.mul_(beta1).add_(gf, alpha=1.0 - beta1)
    vf.mul_(beta2).addcmul_(gf, gf, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2s = (1.0 - beta2 ** step) ** 0.5
    pf.addcdiv_(mf, vf.sqrt().div_(bc2s).add_(eps), value=-lr / bc1)
    p.copy_(pf)
    m.copy_(mf)
    v.copy_(vf)


class FusedAdamW(torch.optim.Optimizer):
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 1e-2,
                 state_dtype: Optional[torch.dtype] = None):
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1:
            raise ValueError("FusedAdamW: lr and eps must be >= 0 and the betas in [0, 1)")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.state_dtype = state_dtype
        self.launches = 0
        for group in self.param_groups:
            # one device-side step record per (param dtype, moment dtype, device) bucket of the group:
            # [steps taken, 1 - beta1^t, sqrt(1 - beta2^t), unused]
            group["step_state"] = {}
            group["host_steps"] = 0
            for p in group["params"]:
                dt = state_dtype or p.dtype
                self.state[p]["exp_avg"] = torch.zeros_like(p, dtype=dt, memory_format=torch.preserve_format)
                self.state[p]["exp_avg_sq"] = torch.zeros_like(p, dtype=dt, memory_format=torch.preserve_format)
                if p.is_cuda:
                    group["step_state"].setdefault((p.dtype, dt, p.device), torch.zeros(4, dtype=torch.float32, device=p.device))

    @staticmethod
    def _native(p, g, m) -> bool:
        return (p.is_cuda and g.is_cuda and p.dtype in _DT and g.dtype == p.dtype and m.dtype in _DT and p.is_contiguous() and g.is_contiguous()
                and not (p.dtype == torch.float32 and m.dtype == torch.bfloat16))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            buckets = {}          # (param dtype, state dtype, device) -> tensors for the kernel
            fallback = []
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if self._native(p, p.grad, st["exp_avg"]):
                    buckets.setdefault((p.dtype, st["exp_avg"].dtype, p.device), []).append(p)
                else:
                    fallback.append(p)
            if fallback:
                group["host_steps"] += 1
                for p in fallback:
                    st = self.state[p]
                    adamw_reference_(p, p.grad, st["exp_avg"], st["exp_avg_sq"], group["host_steps"], group["lr"], beta1, beta2, group["eps"],
                                     group["weight_decay"])
            for (pdt, sdt, dev), plist in buckets.items():
                if not hasattr(lib, "HcclFusedAdamW"):
                    raise RuntimeError("libhccl_b200.so predates the fused optimizer kernel: rebuild it with `python hccl_b200/build.py`")
                table = (_AdamTensor * len(plist))()
                for i, p in enumerate(plist):
                    st = self.state[p]
                    table[i] = _AdamTensor(p.data_ptr(), p.grad.data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(), p.numel())
                step_state = group["step_state"][(pdt, sdt, dev)]
                stream = ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(dev.index if dev.index is not None else torch.cuda.current_device()))
                lr = group["lr"]
                lr_dev = ctypes.c_void_p(lr.data_ptr()) if isinstance(lr, torch.Tensor) and lr.is_cuda else ctypes.c_void_p(0)
                _check(lib.HcclFusedAdamW(table, len(plist), int(_DT[pdt]), int(_DT[sdt]), float(lr) if not isinstance(lr, torch.Tensor) else 0.0, lr_dev,
                                          beta1, beta2, group["eps"], group["weight_decay"], ctypes.c_void_p(step_state.data_ptr()), stream),
                       "HcclFusedAdamW")
                n = int(lib.HcclFusedAdamWLaunches(len(plist)))
                self.launches += n
                _fused._count(n)
        return loss
