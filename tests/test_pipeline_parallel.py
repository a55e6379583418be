"""GPipe schedule on BatchSendRecv (host-engine ranks as stages) against the same model trained in one piece."""
import copy

import pytest
import torch

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200.parallel import gpipe_step

from test_host_engine import run_ranks


@pytest.mark.parametrize("P,n_micro", [(1, 3), (2, 1), (3, 4), (4, 2)])
def test_pipeline_matches_single_process_training(P, n_micro):
    torch.manual_seed(0)
    width, batch = 12, 5
    stages = [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()) for _ in range(P)]
    whole = torch.nn.Sequential(*[copy.deepcopy(s) for s in stages])
    micro = [torch.randn(batch, width) for _ in range(n_micro)]
    targets = [torch.randn(batch, width) for _ in range(n_micro)]
    # reference: the mean loss over micro-batches, gradients accumulated
    ref_loss = 0.0
    for x, t in zip(micro, targets):
        loss = (whole(x) - t).pow(2).mean() / n_micro
        loss.backward()
        ref_loss += loss.item()
    comms = Communicator.host_sim(P, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    losses = [None] * P

    def body(r, c):
        losses[r] = gpipe_step(stages[r], c, n_micro, (batch, width), torch.float32, "cpu", inputs=micro if r == 0 else None,
                               loss_fn=(lambda y, m: (y - targets[m]).pow(2).mean()) if r == P - 1 else None)

    run_ranks(comms, body)
    assert all(l is None for l in losses[:-1])
    assert abs(float(losses[-1]) - ref_loss) < 1e-6
    for r in range(P):
        for p, q in zip(stages[r].parameters(), whole[r].parameters()):
            torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=1e-6)
    for c in comms:
        c.destroy()
