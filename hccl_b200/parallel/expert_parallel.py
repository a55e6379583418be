"""Expert parallelism on the AlltoAll / AlltoAllV operators.

The reference's answer to MoE is its AlltoAll family (41 registered algorithms, hierarchical and pairwise variants;
EP = 64 deployments in docs/en/user_guide/hccl_env/comm_retry_perf_impact.md:37,59-60).  ``moe_forward`` is the
portable user of those operators: it works on any communicator - device ranks or host-engine ranks - and any dtype,
and is what ``hccl_b200.ops.moe.MoeDispatcher`` (the fused dispatch / combine kernels with fp8 block quantisation)
is measured against.

Experts are numbered globally; rank r hosts experts ``[r * E / P, (r + 1) * E / P)``.

1. every (token, k) pair is sorted by expert; one AlltoAll carries the per-expert row counts, so that a receiver
   knows how the rows it gets are grouped;
2. AlltoAllV moves the rows to the ranks of their experts;
3. the local experts run on their rows (one contiguous slice per expert);
4. AlltoAllV brings the outputs back, and the gate weights fold the k outputs of a token together.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


def moe_forward(x: torch.Tensor, topk_idx: torch.Tensor, topk_weight: torch.Tensor, local_experts: Sequence[Callable[[torch.Tensor], torch.Tensor]], comm,
                n_experts: int) -> torch.Tensor:
    """x ``[T, H]``, topk_idx ``[T, K]`` (global expert ids), topk_weight ``[T, K]``; ``local_experts[i]`` is this rank's
    i-th expert, a map ``[rows, H] -> [rows, H]``.  Returns ``[T, H]`` in x's dtype."""
    P, r = comm.world_size, comm.rank
    T, H = x.shape
    K = topk_idx.shape[1]
    if n_experts % P:
        raise ValueError(f"moe_forward: {n_experts} experts do not divide over {P} ranks")
    e_local = n_experts // P
    if len(local_experts) != e_local:
        raise ValueError(f"moe_forward: rank hosts {e_local} experts, got {len(local_experts)}")
    dev = x.device
    flat_e = topk_idx.reshape(-1).long()
    order = torch.argsort(flat_e, stable=True)                   # pairs grouped by expert, hence by destination rank
    rows = x[order // K].contiguous()
    per_expert = torch.bincount(flat_e, minlength=n_experts)     # rows I send to every expert
    # 1. counts: block q of the send buffer = my counts for rank q's experts
    recv_per_expert = torch.empty_like(per_expert)
    if P > 1:
        comm.all_to_all(per_expert.contiguous(), recv_per_expert)
    else:
        recv_per_expert.copy_(per_expert)
    recv_per_expert = recv_per_expert.view(P, e_local)           # [source rank, my expert]
    send_rows = per_expert.view(P, e_local).sum(1).tolist()
    recv_rows = recv_per_expert.sum(1).tolist()

    def exchange(buf, send_counts, recv_counts):
        out = torch.empty((sum(recv_counts), H), dtype=buf.dtype, device=dev)
        if P == 1:
            out.copy_(buf)
            return out
        sc = [c * H for c in send_counts]
        rc = [c * H for c in recv_counts]
        sd = [sum(sc[:i]) for i in range(P)]
        rd = [sum(rc[:i]) for i in range(P)]
        src = buf if buf.numel() else torch.zeros(1, dtype=buf.dtype, device=dev)        # a rank may have nothing to send
        dst = out if out.numel() else torch.zeros(1, dtype=buf.dtype, device=dev)
        comm.all_to_all_v(src, sc, sd, dst, rc, rd)
        return out

    # 2. rows to their experts; they arrive ordered by (source rank, expert)
    got = exchange(rows, send_rows, recv_rows)
    counts = recv_per_expert.reshape(-1).tolist()                # row counts in arrival order
    starts = [0]
    for c in counts:
        starts.append(starts[-1] + c)
    # 3. every local expert takes its slices (one per source rank)
    y = torch.empty_like(got)
    for e in range(e_local):
        pieces = [(starts[q * e_local + e], starts[q * e_local + e + 1]) for q in range(P)]
        idx = torch.cat([torch.arange(b, t, device=dev) for b, t in pieces]) if pieces else torch.empty(0, dtype=torch.long, device=dev)
        if idx.numel():
            y[idx] = local_experts[e](got[idx]).to(y.dtype)
    # 4. outputs back to the owners of the tokens (the counts swap roles), then un-sort and fold with the gate weights
    back = exchange(y, recv_rows, send_rows)
    pair_out = torch.empty((T * K, H), dtype=x.dtype, device=dev)
    pair_out[order] = back
    w = topk_weight.reshape(T, K, 1).to(torch.float32)
    return (pair_out.view(T, K, H).float() * w).sum(1).to(x.dtype)
