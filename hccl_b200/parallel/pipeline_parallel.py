"""Pipeline parallelism on BatchSendRecv.

The reference names Send / Recv / BatchSendRecv as the operators pipeline parallelism introduces
(docs/en/user_guide/hccl_env/comm_retry_perf_impact.md:19; ring example
examples/01_point_to_point/02_batch_send_recv_ring).  ``gpipe_step`` is the thin user: rank r holds stage r of a
model; M micro-batches flow forward through the stages and their gradients flow back (all forwards, then all
backwards - the GPipe schedule).  Activations and gradients move between neighbours with one BatchSendRecv per rank
and tick, which pairs the send of stage r with the receive of stage r + 1 in the same tick.

Every rank makes exactly one BatchSendRecv call per tick, with an empty item list when it has nothing to exchange:
on a host-engine or emulated communicator every rank has to take part in every launch, and on device communicators an
empty batch returns at once.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch


def gpipe_step(stage: torch.nn.Module, comm, n_micro: int, act_shape: Sequence[int], act_dtype: torch.dtype, device,
               inputs: Optional[List[torch.Tensor]] = None, loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None) -> Optional[torch.Tensor]:
    """One training step of a P-stage pipeline (forward and backward of ``n_micro`` micro-batches; parameter gradients
    accumulate in ``stage``).

    ``inputs``: the micro-batches, needed on rank 0 only.  ``loss_fn(output, m)``: scalar loss of micro-batch m, needed on
    the last rank only; the step's loss is the mean over micro-batches.  ``act_shape`` / ``act_dtype``: shape and dtype
    of the tensor that travels between stages (the same at every boundary).  Returns the mean loss on the last rank,
    None elsewhere."""
    P, r = comm.world_size, comm.rank
    first, last = r == 0, r == P - 1
    ticks = n_micro + P - 1
    xs: List[Optional[torch.Tensor]] = [None] * n_micro          # stage inputs, kept for backward
    ys: List[Optional[torch.Tensor]] = [None] * n_micro          # stage outputs (the loss on the last rank)
    recv_buf = torch.empty(tuple(act_shape), dtype=act_dtype, device=device)
    total = torch.zeros((), dtype=torch.float32, device=device)

    def active(rank: int, tick: int) -> bool:
        return 0 <= tick - rank < n_micro

    # ---------------------------------------------------------------- forward: stage r handles micro-batch t - r at tick t
    pending = None                                               # the activation that arrived in the previous tick
    for t in range(ticks):
        out = None
        if active(r, t):
            m = t - r
            x = inputs[m] if first else pending
            x = x.detach().requires_grad_(not first)
            xs[m] = x
            y = stage(x)
            if last:
                loss = loss_fn(y, m) / n_micro
                ys[m] = loss
                total = total + loss.detach().float()
            else:
                ys[m] = y
                out = y.detach().contiguous()
        items = []
        if out is not None:
            items.append(("send", out, r + 1))
        if not first and active(r - 1, t):                       # my left neighbour produced something in this tick
            items.append(("recv", recv_buf, r - 1))
        comm.batch_send_recv(items)
        pending = recv_buf.clone() if (not first and active(r - 1, t)) else None

    # ---------------------------------------------------------------- backward: the last stage starts, micro-batches in reverse
    def b_active(rank: int, tick: int) -> bool:
        return 0 <= tick - (P - 1 - rank) < n_micro

    pending = None
    for t in range(ticks):
        gout = None
        if b_active(r, t):
            m = n_micro - 1 - (t - (P - 1 - r))
            if last:
                ys[m].backward()
            else:
                ys[m].backward(pending)
            if not first:
                gout = xs[m].grad.contiguous()
            xs[m], ys[m] = None, None
        items = []
        if gout is not None:
            items.append(("send", gout, r - 1))
        if not last and b_active(r + 1, t):
            items.append(("recv", recv_buf, r + 1))
        comm.batch_send_recv(items)
        pending = recv_buf.clone() if (not last and b_active(r + 1, t)) else None
    return total if last else None
