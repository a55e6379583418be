"""Expert parallelism on AlltoAll / AlltoAllV (host-engine ranks) against a dense computation that evaluates every
chosen expert locally."""
import pytest
import torch

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200.parallel import moe_forward

from test_host_engine import run_ranks


def make_experts(n_experts, hidden, seed=0):
    g = torch.Generator().manual_seed(seed)
    ws = [torch.randn(hidden, hidden, generator=g) / hidden ** 0.5 for _ in range(n_experts)]
    return [(lambda w: (lambda rows: torch.tanh(rows @ w)))(w) for w in ws]


def dense(x, idx, weight, experts):
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for k in range(idx.shape[1]):
            out[t] += weight[t, k] * experts[int(idx[t, k])](x[t:t + 1])[0]
    return out


@pytest.mark.parametrize("P,n_experts,topk", [(1, 4, 2), (2, 4, 2), (4, 8, 3), (3, 6, 1)])
def test_moe_forward_matches_dense(P, n_experts, topk):
    T, H = 37, 16
    experts = make_experts(n_experts, H)
    e_local = n_experts // P
    xs, idxs, ws = [], [], []
    for r in range(P):
        g = torch.Generator().manual_seed(50 + r)
        xs.append(torch.randn(T, H, generator=g))
        # distinct experts per token, skewed so that some experts get nothing from some ranks
        idxs.append(torch.stack([torch.randperm(n_experts, generator=g)[:topk] for _ in range(T)]).int() if r % 2 == 0
                    else torch.zeros(T, topk, dtype=torch.int32) + torch.arange(topk, dtype=torch.int32))
        ws.append(torch.softmax(torch.randn(T, topk, generator=g), dim=-1))
    comms = Communicator.host_sim(P, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    outs = [None] * P

    def body(r, c):
        outs[r] = moe_forward(xs[r], idxs[r], ws[r], experts[r * e_local:(r + 1) * e_local], c, n_experts)

    run_ranks(comms, body)
    for r in range(P):
        torch.testing.assert_close(outs[r], dense(xs[r], idxs[r], ws[r], experts), rtol=1e-5, atol=1e-5)
    for c in comms:
        c.destroy()


def test_argument_checks():
    comms = Communicator.host_sim(3)
    x = torch.zeros(2, 4)
    with pytest.raises(ValueError):
        moe_forward(x, torch.zeros(2, 1, dtype=torch.int32), torch.ones(2, 1), [], comms[0], 4)        # 4 experts over 3 ranks
    with pytest.raises(ValueError):
        moe_forward(x, torch.zeros(2, 1, dtype=torch.int32), torch.ones(2, 1), [], comms[0], 6)        # two local experts expected
    for c in comms:
        c.destroy()
