"""Reductions fused with a cast and a scale, the ring and halving-doubling device templates and the AlltoAll that
lands in the receivers' slabs - ranks emulated on one GPU, results against fp64 references."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

import hccl_b200 as hb
from hccl_b200 import Communicator, ReduceOp
from hccl_b200._lib import lib


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(n, device="cuda", generator=g, dtype=torch.float32) * 2 - 1).to(dtype)


@pytest.fixture(scope="module", params=[2, 4, 8])
def comms(request):
    torch.cuda.set_device(0)
    cs = Communicator.emulated(request.param, hb.make_config(buffer_mib=16))
    yield cs
    torch.cuda.synchronize()
    for c in cs:
        c.destroy()


class _Algo:
    """HCCL_ALGO for the duration of a block (the environment is parsed once per process unless reloaded)."""

    def __init__(self, value):
        self.value = value

    def __enter__(self):
        self.old = os.environ.get("HCCL_ALGO")
        os.environ["HCCL_ALGO"] = self.value
        lib.HcclReloadEnvConfig()

    def __exit__(self, *a):
        if self.old is None:
            os.environ.pop("HCCL_ALGO", None)
        else:
            os.environ["HCCL_ALGO"] = self.old
        lib.HcclReloadEnvConfig()


PAIRS = [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32), (torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
         (torch.float16, torch.float32)]


@pytest.mark.parametrize("tin,tout", PAIRS)
@pytest.mark.parametrize("n", [5, 4096, 70001, 3 * 1024 * 1024 + 8])
def test_all_reduce_with_cast_and_average(comms, tin, tout, n):
    p = len(comms)
    ins = [_rand(n, tin, 10 + r) for r in range(p)]
    outs = [torch.empty(n, device="cuda", dtype=tout) for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.all_reduce_ex(x, y, ReduceOp.SUM, scale=1.0 / p)
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    assert comms[0].last_algorithm().endswith("Cast")
    ref = torch.stack([x.double() for x in ins]).mean(0)
    tol = 1e-2 if tout != torch.float32 else (1e-6 if tin == torch.float32 else 1e-6)
    for y in outs:
        torch.testing.assert_close(y.double(), ref, rtol=tol, atol=tol)
    for y in outs[1:]:
        assert torch.equal(y.view(torch.uint8), outs[0].view(torch.uint8))


@pytest.mark.parametrize("tin,tout", PAIRS[:3])
@pytest.mark.parametrize("n", [8, 5000, 300000])
def test_reduce_scatter_with_cast_and_scale(comms, tin, tout, n):
    p = len(comms)
    ins = [_rand(n * p, tin, 30 + r) for r in range(p)]
    outs = [torch.empty(n, device="cuda", dtype=tout) for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.reduce_scatter_ex(x, y, ReduceOp.SUM, scale=0.5)
    torch.cuda.synchronize()
    ref = torch.stack([x.double() for x in ins]).sum(0) * 0.5
    tol = 1e-2 if tout != torch.float32 else 1e-6
    for r, y in enumerate(outs):
        torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=tol, atol=tol * p)


def test_cast_in_place_on_symmetric_memory(comms):
    """Averaging in place (same type) on buffers from comm.empty: the gradient-bucket case."""
    p = len(comms)
    for n in (1000, 200000):
        xs = [c.empty((n,), torch.float32) for c in comms]
        src = [_rand(n, torch.float32, 60 + r) for r in range(p)]
        for x, s in zip(xs, src):
            x.copy_(s)
        for c, x in zip(comms, xs):
            c.all_reduce_ex(x, scale=1.0 / p)
        torch.cuda.synchronize()
        ref = torch.stack([s.double() for s in src]).mean(0)
        for x in xs:
            torch.testing.assert_close(x.double(), ref, rtol=1e-6, atol=1e-6)
        for c, x in zip(comms, xs):
            c.free(x)


@pytest.mark.parametrize("n", [16, 4099, 250000])
def test_ring_reduce_scatter_and_all_gather(comms, n):
    p = len(comms)
    with _Algo("reducescatter=level0:ring/allgather=level0:ring"):
        for dtype in (torch.float32, torch.bfloat16):
            ins = [_rand(n * p, dtype, 80 + r) for r in range(p)]
            outs = [torch.empty(n, device="cuda", dtype=dtype) for _ in range(p)]
            for rep in range(2):
                for c, x, y in zip(comms, ins, outs):
                    c.reduce_scatter(x, y)
                torch.cuda.synchronize()
                assert comms[0].last_algorithm() == "P2pReduceScatterSoleRing"
                ref = torch.stack([x.double() for x in ins]).sum(0)
                tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
                for r, y in enumerate(outs):
                    torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=tol, atol=tol * p)
            gin = [_rand(n, dtype, 90 + r) for r in range(p)]
            gout = [torch.empty(n * p, device="cuda", dtype=dtype) for _ in range(p)]
            for c, x, y in zip(comms, gin, gout):
                c.all_gather(x, y)
            torch.cuda.synchronize()
            assert comms[0].last_algorithm() == "P2pAllGatherSoleRing"
            for y in gout:
                assert torch.equal(y, torch.cat(gin))
    assert comms[0].async_error() == hb.Result.SUCCESS


@pytest.mark.parametrize("n", [8, 4099, 1 << 20])
def test_halving_doubling_all_reduce(comms, n):
    p = len(comms)
    with _Algo("allreduce=level0:H-D_R"):
        for inplace in (False, True):
            ins = [_rand(n, torch.float32, 120 + r) for r in range(p)]
            ref = torch.stack([x.double() for x in ins]).sum(0)
            outs = ins if inplace else [torch.empty_like(x) for x in ins]
            for c, x, y in zip(comms, ins, outs):
                c.all_reduce(x, y)
            torch.cuda.synchronize()
            assert comms[0].last_algorithm() == "P2pAllReduceSoleRhd"
            for y in outs:
                torch.testing.assert_close(y.double(), ref, rtol=1e-5, atol=1e-5)
            for y in outs[1:]:
                assert torch.equal(y, outs[0])
    assert comms[0].async_error() == hb.Result.SUCCESS


@pytest.mark.parametrize("per", [70000, 300000])
def test_all_to_all_through_the_slabs(comms, per):
    """Blocks too large for flag-in-data lines and small enough for the landing zone: posted writes and one barrier;
    several in a row reuse both landing copies."""
    p = len(comms)
    for rep in range(3):
        ins = [_rand(per * p, torch.float32, 200 + 10 * rep + r) for r in range(p)]
        outs = [torch.empty(per * p, device="cuda") for _ in range(p)]
        for c, x, y in zip(comms, ins, outs):
            c.all_to_all(x, y)
        torch.cuda.synchronize()
        if per * 4 * p * 2 + 64 * p <= 7 << 20:
            assert comms[0].last_algorithm() == "P2pAlltoAllSoleMeshPush", comms[0].last_algorithm()
        for r in range(p):
            for q in range(p):
                assert torch.equal(outs[r][q * per:(q + 1) * per], ins[q][r * per:(r + 1) * per])
    assert comms[0].async_error() == hb.Result.SUCCESS


def _push_or_switch(name, push):
    # with a switch that reduces, the staged switch form may still price below the push form; both are legal here
    # ... and blocks that still fit the flag-in-data lines take those
    return name == push or name.startswith("Nvls") or name.endswith("LL")


@pytest.mark.parametrize("n", [70000, 300000, 1 << 20])
def test_reduce_scatter_of_ordinary_buffers_without_staging(comms, n):
    """Ordinary tensors, blocks pushed into the receivers' landing copies; blocks of 4 MiB need several launches with
    this slab; out of place and in place (the output is this rank's block of the input)."""
    p = len(comms)
    for dtype in (torch.float32, torch.bfloat16):
        for inplace in (False, True):
            ins = [_rand(n * p, dtype, 300 + r) for r in range(p)]
            ref = torch.stack([x.double() for x in ins]).sum(0)
            outs = [x[r * n:(r + 1) * n] for r, x in enumerate(ins)] if inplace else [torch.empty(n, device="cuda", dtype=dtype) for _ in range(p)]
            for c, x, y in zip(comms, ins, outs):
                c.reduce_scatter(x, y)
            torch.cuda.synchronize()
            assert _push_or_switch(comms[0].last_algorithm(), "P2pReduceScatterSoleMeshPush"), comms[0].last_algorithm()
            tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
            for r, y in enumerate(outs):
                torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=tol, atol=tol * p)
    assert comms[0].async_error() == hb.Result.SUCCESS


@pytest.mark.parametrize("n", [70001, 1 << 20, 3 * 1024 * 1024 + 8])
def test_all_reduce_of_ordinary_buffers_without_staging(comms, n):
    p = len(comms)
    with _Algo("allreduce=level0:twoshot"):
        for inplace in (False, True):
            ins = [_rand(n, torch.float32, 340 + r) for r in range(p)]
            ref = torch.stack([x.double() for x in ins]).sum(0)
            outs = ins if inplace else [torch.empty_like(x) for x in ins]
            for c, x, y in zip(comms, ins, outs):
                c.all_reduce(x, y)
            torch.cuda.synchronize()
            assert comms[0].last_algorithm() == "P2pAllReduceSoleMeshPushTwoShot", comms[0].last_algorithm()
            for y in outs:
                torch.testing.assert_close(y.double(), ref, rtol=1e-5, atol=1e-5)
            for y in outs[1:]:
                assert torch.equal(y, outs[0])
    assert comms[0].async_error() == hb.Result.SUCCESS


def test_push_forms_of_different_shapes_back_to_back(comms):
    """The landing copies are taken in turn by a count of push operators, not by block row: operators of different
    sizes and grids follow one another without a barrier between them and never write a copy that is still read."""
    p = len(comms)
    shapes = [70000, 300000, 90000, 1 << 19, 66000, 300000]
    cases = []
    for i, n in enumerate(shapes):
        rs_in = [_rand(n * p, torch.float32, 400 + 10 * i + r) for r in range(p)]
        rs_out = [torch.empty(n, device="cuda") for _ in range(p)]
        a2a_in = [_rand(n * p, torch.float32, 500 + 10 * i + r) for r in range(p)]
        a2a_out = [torch.empty(n * p, device="cuda") for _ in range(p)]
        cases.append((n, rs_in, rs_out, a2a_in, a2a_out))
    for n, rs_in, rs_out, a2a_in, a2a_out in cases:          # all launches first, one synchronize at the end
        for c, x, y in zip(comms, rs_in, rs_out):
            c.reduce_scatter(x, y)
        if n * 4 * p * 2 + 64 * p <= 7 << 20:
            for c, x, y in zip(comms, a2a_in, a2a_out):
                c.all_to_all(x, y)
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    for n, rs_in, rs_out, a2a_in, a2a_out in cases:
        ref = torch.stack([x.double() for x in rs_in]).sum(0)
        for r, y in enumerate(rs_out):
            torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=1e-5, atol=1e-5)
        if n * 4 * p * 2 + 64 * p <= 7 << 20:
            for r in range(p):
                for q in range(p):
                    assert torch.equal(a2a_out[r][q * n:(q + 1) * n], a2a_in[q][r * n:(r + 1) * n])


@pytest.mark.parametrize("n", [(4 << 20) // 4 + 4, 5 * 1024 * 1024 + 12])
def test_pipelined_broadcast(comms, n):
    """Scatter from the root and AllGather among the others, piece by piece: ordinary buffers (pieces wait in the
    exchange region, several launches with this slab) and symmetric buffers (peers read the buffers themselves)."""
    p = len(comms)
    if p < 3:
        pytest.skip("one receiver pulls everything from the root")
    with _Algo("broadcast=level0:pipeline"):
        for sym in (False, True):
            for root in (0, p - 1):
                src = _rand(n, torch.float32, 600 + root)
                bufs = [c.empty((n,), torch.float32) if sym else torch.empty(n, device="cuda") for c in comms]
                for r, x in enumerate(bufs):
                    x.copy_(src) if r == root else x.fill_(-1.0)
                for c, x in zip(comms, bufs):
                    c.broadcast(x, root)
                torch.cuda.synchronize()
                assert comms[0].last_algorithm() == "P2pBroadcastSoleMeshPipe", comms[0].last_algorithm()
                for x in bufs:
                    assert torch.equal(x, src)
                if sym:
                    for c, x in zip(comms, bufs):
                        c.free(x)
    assert comms[0].async_error() == hb.Result.SUCCESS
