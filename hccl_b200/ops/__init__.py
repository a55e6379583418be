"""Operators on tensors: MC2 fused matmul + collective, MoE dispatch / combine and the
torch.distributed-style functional collectives."""
from . import functional, mc2, moe  # noqa: F401
from .optim import FusedAdamW  # noqa: F401
