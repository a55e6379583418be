"""Calls whose buffers differ from rank to rank, AlltoAllV larger than the staging slab, in-place reductions on
symmetric memory and runs of small broadcasts - ranks emulated on one GPU, results against plain PyTorch references."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import hccl_b200 as hb
from hccl_b200 import Communicator, ReduceOp


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(n, device="cuda", generator=g, dtype=torch.float32) * 2 - 1).to(dtype)


@pytest.fixture(scope="module", params=[2, 4, 8])
def comms(request):
    torch.cuda.set_device(0)
    cs = Communicator.emulated(request.param, hb.make_config(buffer_mib=8))
    yield cs
    torch.cuda.synchronize()
    for c in cs:
        c.destroy()


@pytest.mark.parametrize("n", [1000, 70000, 3 * 1024 * 1024])
def test_one_rank_unaligned_the_others_aligned(comms, n):
    """One rank passes a 4-byte aligned view, the others 16-byte aligned tensors: all ranks must end up with the same
    algorithm and launch shape (the facts they do not all share are dropped), and with the right sum."""
    p = len(comms)
    base = [_rand(n + 4, torch.float32, 50 + r) for r in range(p)]
    ins = [b[1:1 + n] if r == 1 else b[:n] for r, b in enumerate(base)]
    outs = [torch.empty(n + 4, device="cuda")[(1 if r == 1 else 0):][:n] for r in range(p)]
    ref = torch.stack([x.double() for x in ins]).sum(0)
    for c, x, y in zip(comms, ins, outs):
        c.all_reduce(x, y)
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    assert len({c.last_algorithm() for c in comms}) == 1
    for y in outs:
        torch.testing.assert_close(y.double(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n", [4096, 300000])
def test_one_rank_symmetric_the_others_plain(comms, n):
    """A buffer from comm.empty on one rank only: nobody may read it in place on the peers (the peers have no such
    buffer at that offset), so the call is staged everywhere."""
    p = len(comms)
    sym = [c.empty((n,), torch.float32) for c in comms]           # collective allocation; only rank 0 uses its buffer
    ins = [_rand(n, torch.float32, 90 + r) for r in range(p)]
    sym[0].copy_(ins[0])
    outs = [torch.empty(n, device="cuda") for _ in range(p)]
    for r, (c, y) in enumerate(zip(comms, outs)):
        c.all_reduce(sym[0] if r == 0 else ins[r], y)
    torch.cuda.synchronize()
    ref = torch.stack([x.double() for x in ins]).sum(0)
    for y in outs:
        torch.testing.assert_close(y.double(), ref, rtol=1e-5, atol=1e-5)
    # all_gather the same way
    outs = [torch.empty(n * p, device="cuda") for _ in range(p)]
    for r, (c, y) in enumerate(zip(comms, outs)):
        c.all_gather(sym[0] if r == 0 else ins[r], y)
    torch.cuda.synchronize()
    for y in outs:
        assert torch.equal(y, torch.cat(ins))
    for c, s in zip(comms, sym):
        c.free(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [8, 1024, 20000, 200000, 2 * 1024 * 1024])
def test_all_reduce_in_place_on_symmetric_memory(comms, dtype, n):
    """x = all_reduce(x) with x from comm.empty at sizes that select the flag-in-data, one-shot and two-shot forms:
    a rank must not overwrite its input while a peer still reads it."""
    p = len(comms)
    xs = [c.empty((n,), dtype) for c in comms]
    src = [_rand(n, dtype, 500 + r) for r in range(p)]
    ref = torch.stack([s.double() for s in src]).sum(0)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
    for rep in range(3):
        for x, s in zip(xs, src):
            x.copy_(s)
        for c, x in zip(comms, xs):
            c.all_reduce(x)
        torch.cuda.synchronize()
        for x in xs:
            torch.testing.assert_close(x.double(), ref, rtol=tol, atol=tol * p)
        for x in xs[1:]:
            assert torch.equal(x.view(torch.uint8), xs[0].view(torch.uint8))
    for c, x in zip(comms, xs):
        c.free(x)


def test_all_to_all_v_four_times_the_staging_slab(comms):
    """Ordinary (unregistered) buffers whose pairs are far larger than a pair's staging window: the kernel derives the
    number of passes from all ranks' counts.  Counts differ per pair, one pair is empty."""
    p = len(comms)
    unit = (8 << 20) // p            # elements of 4 bytes: a pair of `unit` elements is 4x its window share of an 8 MiB slab
    send_counts = [[0 if (r == 0 and q == p - 1) else unit // 2 + 1000 * ((r + 2 * q) % 5) + 3 for q in range(p)] for r in range(p)]
    recv_counts = [[send_counts[q][r] for q in range(p)] for r in range(p)]
    sd = [[sum(send_counts[r][:q]) for q in range(p)] for r in range(p)]
    rd = [[sum(recv_counts[r][:q]) for q in range(p)] for r in range(p)]
    ins = [_rand(sum(send_counts[r]), torch.float32, 700 + r) for r in range(p)]
    outs = [torch.zeros(sum(recv_counts[r]), device="cuda") for r in range(p)]
    for r, c in enumerate(comms):
        c.all_to_all_v(ins[r], send_counts[r], sd[r], outs[r], recv_counts[r], rd[r])
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    for r in range(p):
        for q in range(p):
            want = ins[q][sd[q][r]:sd[q][r] + send_counts[q][r]]
            got = outs[r][rd[r][q]:rd[r][q] + recv_counts[r][q]]
            assert torch.equal(got, want), f"block {q}->{r}"
    # a small one right after (one pass) reuses the protocol state
    small = [[17 + r + q for q in range(p)] for r in range(p)]
    rsmall = [[small[q][r] for q in range(p)] for r in range(p)]
    ssd = [[sum(small[r][:q]) for q in range(p)] for r in range(p)]
    rrd = [[sum(rsmall[r][:q]) for q in range(p)] for r in range(p)]
    outs2 = [torch.zeros(sum(rsmall[r]), device="cuda") for r in range(p)]
    for r, c in enumerate(comms):
        c.all_to_all_v(ins[r], small[r], ssd[r], outs2[r], rsmall[r], rrd[r])
    torch.cuda.synchronize()
    for r in range(p):
        for q in range(p):
            assert torch.equal(outs2[r][rrd[r][q]:rrd[r][q] + rsmall[r][q]], ins[q][ssd[q][r]:ssd[q][r] + small[q][r]])


def test_runs_of_small_broadcasts_and_mixed_small_ops(comms):
    """Many flag-in-data operators in a row with changing roots: the line slots are reused every second operator, so
    each result depends on the credit that keeps a writer from running over lines that were not read yet."""
    p = len(comms)
    n = 2048
    for it in range(12):
        root = it % p
        bufs = [_rand(n, torch.float32, 900 + it) if r == root else torch.zeros(n, device="cuda") for r in range(p)]
        want = bufs[root].clone()
        for c, b in zip(comms, bufs):
            c.broadcast(b, root)
        if it % 3 == 2:
            xs = [_rand(n, torch.float32, 950 + it + r) for r in range(p)]
            ref = torch.stack(xs).sum(0)
            for c, x in zip(comms, xs):
                c.all_reduce(x)
        torch.cuda.synchronize()
        for b in bufs:
            assert torch.equal(b, want)
        if it % 3 == 2:
            for x in xs:
                torch.testing.assert_close(x, ref, rtol=1e-5, atol=1e-5)
    assert comms[0].async_error() == hb.Result.SUCCESS
