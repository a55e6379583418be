"""Long-sequence attention across ranks, built from the operators only.

The reference ships no context-parallel code: its documents name the collectives such schemes consume (AlltoAll for
the head / sequence exchange, Send / Recv rings for blockwise attention; CP = 16 appears as a deployment example in
docs/en/user_guide/hccl_env/comm_retry_perf_impact.md:36).  These two functions are the thin users of those
operators, for sequences sharded over the ranks of a communicator:

* ``ulysses_attention``: two AlltoAll calls turn the sequence shard ``[S / P, H, D]`` into a head shard
  ``[S, H / P, D]`` and back; attention itself is local and sees the whole sequence.
* ``ring_attention``: keys and values travel once around the ring with BatchSendRecv (P - 1 steps) while every rank
  folds one block per step into its running softmax (the log-sum-exp merge of blockwise attention).

Tensors may be CUDA tensors on a device communicator or CPU tensors on a host-engine communicator (ranks as threads),
which is how the tests run them without a GPU.  ``causal=True`` assumes that rank r holds the r-th contiguous slice
of the sequence.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def _sdpa(q, k, v, causal: bool, scale: float):
    # [S, H, D] -> [H, S, D]
    out = F.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), is_causal=causal, scale=scale)
    return out.transpose(0, 1).contiguous()


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm, causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """q, k, v: this rank's sequence shard ``[S / P, H, D]`` with H divisible by P.  Returns the attention output for
    the same shard.  Four AlltoAll calls (q, k, v in; the output back)."""
    P = comm.world_size
    s, H, D = q.shape
    if H % P:
        raise ValueError(f"ulysses_attention: {H} heads do not divide over {P} ranks")
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if P == 1:
        return _sdpa(q, k, v, causal, scale)
    hp = H // P

    def to_heads(x):
        # block j of the send buffer = my sequence slice of the heads that rank j will own
        send = x.reshape(s, P, hp, D).permute(1, 0, 2, 3).contiguous()
        recv = torch.empty_like(send)
        comm.all_to_all(send, recv)
        # block j of what arrives = rank j's sequence slice of MY heads: concatenating the blocks restores sequence order
        return recv.reshape(P * s, hp, D)

    qh, kh, vh = to_heads(q), to_heads(k), to_heads(v)
    oh = _sdpa(qh, kh, vh, causal, scale)                       # [S, H / P, D], the whole sequence for my heads
    send = oh.reshape(P, s, hp, D).contiguous()                 # block j = rank j's sequence slice
    recv = torch.empty_like(send)
    comm.all_to_all(send, recv)
    return recv.permute(1, 0, 2, 3).reshape(s, H, D).contiguous()   # block j = heads of rank j for my slice


def _block_attention(q, k, v, scale: float, mask: Optional[torch.Tensor]):
    """One block of keys: returns (unnormalised output [s, H, D] in fp32, row maximum [s, H], row sum [s, H])."""
    logits = torch.einsum("shd,thd->sht", q.float(), k.float()) * scale
    if mask is not None:
        logits = logits.masked_fill(~mask[:, None, :], float("-inf"))
    m = logits.amax(dim=-1)
    m_safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)        # a fully masked row contributes nothing
    p = torch.exp(logits - m_safe[..., None])
    return torch.einsum("sht,thd->shd", p, v.float()), m, p.sum(dim=-1)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, comm, causal: bool = False, scale: Optional[float] = None) -> torch.Tensor:
    """q, k, v: this rank's sequence shard ``[S / P, H, D]`` (k and v may have fewer heads than q only if already
    expanded by the caller).  Keys and values move to the right neighbour P - 1 times; the result equals attention
    over the whole sequence."""
    P, r = comm.world_size, comm.rank
    s, H, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    acc = torch.zeros(s, H, D, dtype=torch.float32, device=q.device)
    row_max = torch.full((s, H), float("-inf"), dtype=torch.float32, device=q.device)
    row_sum = torch.zeros(s, H, dtype=torch.float32, device=q.device)
    kv = torch.stack([k, v]).contiguous()
    nxt = torch.empty_like(kv)
    pos_q = torch.arange(s, device=q.device)
    for step in range(P):
        owner = (r - step) % P                                  # whose keys I hold in this step
        if not causal or owner <= r:
            mask = None
            if causal and owner == r:
                mask = pos_q[:, None] >= pos_q[None, :]         # the diagonal block: lower triangle
            out, m, l = _block_attention(q, kv[0], kv[1], scale, mask)
            new_max = torch.maximum(row_max, m)
            safe = torch.where(torch.isinf(new_max), torch.zeros_like(new_max), new_max)
            a_old = torch.exp(torch.where(torch.isinf(row_max), torch.full_like(row_max, float("-inf")), row_max - safe))
            a_new = torch.exp(torch.where(torch.isinf(m), torch.full_like(m, float("-inf")), m - safe))
            acc = acc * a_old[..., None] + out * a_new[..., None]
            row_sum = row_sum * a_old + l * a_new
            row_max = new_max
        if step + 1 < P:
            # stream-ordered on a device communicator: the math above has read kv before it is sent, and the next
            # step's math reads nxt after it has arrived
            comm.batch_send_recv([("send", kv, (r + 1) % P), ("recv", nxt, (r - 1) % P)])
            kv, nxt = nxt, kv
    return (acc / row_sum[..., None]).to(q.dtype)
