"""GradientBucketer: replicated models on host-engine ranks end with the average of their gradients, with and
without the backward hooks, whatever the bucket size."""
import copy

import pytest
import torch

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200.parallel import GradientBucketer

from test_host_engine import run_ranks


def make_model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(16, 32), torch.nn.Tanh(), torch.nn.Linear(32, 32), torch.nn.Tanh(), torch.nn.Linear(32, 4))


@pytest.mark.parametrize("overlap", [False, True])
@pytest.mark.parametrize("bucket_mib", [25.0, 0.001])          # one bucket / one bucket per tensor or two
def test_gradients_are_averaged_across_ranks(overlap, bucket_mib):
    n = 3
    base = make_model()
    models = [copy.deepcopy(base) for _ in range(n)]
    xs = [torch.randn(8, 16, generator=torch.Generator().manual_seed(10 + r)) for r in range(n)]
    # the expected average, computed on one model
    want = [torch.zeros_like(p) for p in base.parameters()]
    for r in range(n):
        m = copy.deepcopy(base)
        m(xs[r]).pow(2).mean().backward()
        for w, p in zip(want, m.parameters()):
            w += p.grad / n
    comms = Communicator.host_sim(n, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    buckets = [None] * n

    def body(r, c):
        b = GradientBucketer(models[r].parameters(), c, bucket_mib=bucket_mib, overlap=overlap)
        buckets[r] = len(b.buckets)
        for _ in range(2):                                          # a second step reuses the buckets
            models[r].zero_grad(set_to_none=True)
            models[r](xs[r]).pow(2).mean().backward()
            b.finish() if overlap else b.reduce()
        b.remove_hooks()

    run_ranks(comms, body)
    assert buckets[0] == (1 if bucket_mib > 1 else 6) or buckets[0] > 1
    for m in models:
        for p, w in zip(m.parameters(), want):
            torch.testing.assert_close(p.grad, w, rtol=1e-5, atol=1e-6)
    for c in comms:
        c.destroy()


def test_unused_parameter_contributes_zeros():
    n = 2
    comms = Communicator.host_sim(n, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    ps = [[torch.nn.Parameter(torch.ones(5)), torch.nn.Parameter(torch.ones(3))] for _ in range(n)]

    def body(r, c):
        b = GradientBucketer(ps[r], c, overlap=True)
        (ps[r][0] * (r + 1)).sum().backward()           # the second parameter takes no part
        b.finish()

    run_ranks(comms, body)
    for r in range(n):
        assert torch.all(ps[r][0].grad == 1.5) and torch.all(ps[r][1].grad == 0)
    for c in comms:
        c.destroy()


def test_sharded_optimizer_matches_replicated_training():
    """ReduceScatter + shard update + AllGather gives the same parameters as averaging the gradients and running the
    same optimizer on the whole model."""
    from hccl_b200.parallel import ShardedOptimizer

    n, steps = 3, 4
    base = make_model()
    xs = [[torch.randn(8, 16, generator=torch.Generator().manual_seed(100 * s + r)) for r in range(n)] for s in range(steps)]
    # the replicated reference
    ref = copy.deepcopy(base)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    for s in range(steps):
        grads = [torch.zeros_like(p) for p in ref.parameters()]
        for r in range(n):
            m = copy.deepcopy(ref)
            m(xs[s][r]).pow(2).mean().backward()
            for g, p in zip(grads, m.parameters()):
                g += p.grad / n
        for p, g in zip(ref.parameters(), grads):
            p.grad = g
        ref_opt.step()
    models = [copy.deepcopy(base) for _ in range(n)]
    comms = Communicator.host_sim(n, None, hb.make_config(buffer_mib=8, exec_timeout_ms=20000))
    shard_sizes = [None] * n

    def body(r, c):
        opt = ShardedOptimizer(models[r].parameters(), c, lambda ps: torch.optim.AdamW(ps, lr=1e-2, weight_decay=0.01))
        shard_sizes[r] = opt.shard.numel()
        for s in range(steps):
            opt.zero_grad()
            models[r](xs[s][r]).pow(2).mean().backward()
            opt.step()

    run_ranks(comms, body)
    total = sum(p.numel() for p in base.parameters())
    assert shard_sizes[0] == (total + n - 1) // n            # each rank holds optimizer state for a third of the model
    for m in models:
        for p, q in zip(m.parameters(), ref.parameters()):
            torch.testing.assert_close(p, q, rtol=1e-4, atol=1e-5)
    for c in comms:
        c.destroy()
