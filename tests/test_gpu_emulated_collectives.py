"""Device collectives with R ranks emulated on ONE GPU: every operator runs as a
single cooperative kernel over all ranks' data, so the full flag protocol
(barriers, LL lines, epochs) is exercised without a second GPU.  Each result is
compared with a plain PyTorch fp32/fp64 reference of the same operator."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

import hccl_b200 as hb
from hccl_b200 import Communicator, ReduceOp


@pytest.fixture(scope="module", params=[2, 4, 8])
def comms(request):
    torch.cuda.set_device(0)
    cs = Communicator.emulated(request.param, hb.make_config(buffer_mib=32))
    yield cs
    torch.cuda.synchronize()
    for c in cs:
        c.destroy()


def _rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.rand(n, device="cuda", generator=g, dtype=torch.float32) * 2 - 1).to(dtype)
    return torch.randint(-50, 50, (n,), device="cuda", generator=g, dtype=torch.int64).to(dtype)


def _tol(dtype):
    return {torch.bfloat16: 3e-2, torch.float16: 4e-3}.get(dtype, 1e-5)


SIZES = [1, 7, 1024, 4099, 65536, 300001, 2 * 1024 * 1024 + 3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16, torch.int32, torch.int64, torch.float64, torch.int8])
@pytest.mark.parametrize("n", SIZES)
def test_all_reduce_sum(comms, dtype, n):
    p = len(comms)
    ins = [_rand(n, dtype, 100 + r) for r in range(p)]
    outs = [torch.empty_like(x) for x in ins]
    for c, x, y in zip(comms, ins, outs):
        c.all_reduce(x, y, ReduceOp.SUM)
    torch.cuda.synchronize()
    ref = torch.stack([x.double() for x in ins]).sum(0)
    for y in outs:
        if dtype.is_floating_point:
            torch.testing.assert_close(y.double(), ref, rtol=_tol(dtype), atol=_tol(dtype) * p)
        else:
            assert torch.equal(y.long(), ref.long().to(dtype).long())
    # every rank must hold bitwise the same result (fixed reduction order)
    for y in outs[1:]:
        assert torch.equal(y.view(torch.uint8), outs[0].view(torch.uint8))
    assert comms[0].async_error() == hb.Result.SUCCESS


@pytest.mark.parametrize("op", [ReduceOp.MAX, ReduceOp.MIN, ReduceOp.PROD])
@pytest.mark.parametrize("n", [5, 4096, 70001])
def test_all_reduce_other_ops(comms, op, n):
    p = len(comms)
    ins = [(_rand(n, torch.float32, 7 + r) * 0.5 + 1.0) for r in range(p)]
    outs = [torch.empty_like(x) for x in ins]
    for c, x, y in zip(comms, ins, outs):
        c.all_reduce(x, y, op)
    torch.cuda.synchronize()
    st = torch.stack(ins)
    ref = {ReduceOp.MAX: st.max(0).values, ReduceOp.MIN: st.min(0).values, ReduceOp.PROD: st.double().prod(0).float()}[op]
    for y in outs:
        torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("n", [3, 1000, 100003])
def test_all_reduce_in_place_and_unaligned(comms, n):
    p = len(comms)
    base = [_rand(n + 5, torch.float32, 40 + r) for r in range(p)]
    views = [b[1:1 + n] for b in base]          # 4-byte aligned only
    ref = torch.stack([v.double() for v in views]).sum(0)
    for c, v in zip(comms, views):
        c.all_reduce(v)
    torch.cuda.synchronize()
    for v in views:
        torch.testing.assert_close(v.double(), ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.uint8])
@pytest.mark.parametrize("n", [1, 33, 4096, 100001])
def test_all_gather(comms, dtype, n):
    p = len(comms)
    ins = [_rand(n, dtype, 200 + r) if dtype != torch.uint8 else torch.randint(0, 255, (n,), device="cuda", dtype=torch.uint8) for r in range(p)]
    outs = [torch.empty(n * p, device="cuda", dtype=dtype) for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.all_gather(x, y)
    torch.cuda.synchronize()
    ref = torch.cat(ins)
    for y in outs:
        assert torch.equal(y.view(torch.uint8), ref.view(torch.uint8))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 33, 4096, 100001])
def test_reduce_scatter(comms, dtype, n):
    p = len(comms)
    ins = [_rand(n * p, dtype, 300 + r) for r in range(p)]
    outs = [torch.empty(n, device="cuda", dtype=dtype) for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.reduce_scatter(x, y)
    torch.cuda.synchronize()
    ref = torch.stack([x.double() for x in ins]).sum(0)
    for r, y in enumerate(outs):
        torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=_tol(dtype), atol=_tol(dtype) * p)


@pytest.mark.parametrize("n", [1, 1000, 200003])
@pytest.mark.parametrize("root", [0, 1])
def test_broadcast_reduce_scatter_root(comms, n, root):
    p = len(comms)
    bufs = [_rand(n, torch.float32, 400 + r) for r in range(p)]
    want = bufs[root].clone()
    for c, b in zip(comms, bufs):
        c.broadcast(b, root)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b, want)
    # reduce
    ins = [_rand(n, torch.float32, 500 + r) for r in range(p)]
    out = torch.zeros(n, device="cuda")
    for r, (c, x) in enumerate(zip(comms, ins)):
        c.reduce(x, out if r == root else None, root)
    torch.cuda.synchronize()
    torch.testing.assert_close(out.double(), torch.stack([x.double() for x in ins]).sum(0), rtol=1e-5, atol=1e-5)
    # scatter
    src = _rand(n * p, torch.float32, 600)
    outs = [torch.empty(n, device="cuda") for _ in range(p)]
    for r, (c, y) in enumerate(zip(comms, outs)):
        c.scatter(src if r == root else None, y, root)
    torch.cuda.synchronize()
    for r, y in enumerate(outs):
        assert torch.equal(y, src[r * n:(r + 1) * n])


@pytest.mark.parametrize("n", [1, 513, 65537])
def test_all_to_all_family(comms, n):
    p = len(comms)
    ins = [_rand(n * p, torch.float32, 700 + r) for r in range(p)]
    outs = [torch.empty(n * p, device="cuda") for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.all_to_all(x, y)
    torch.cuda.synchronize()
    for r in range(p):
        for q in range(p):
            assert torch.equal(outs[r][q * n:(q + 1) * n], ins[q][r * n:(r + 1) * n])
    # variable counts: rank i sends (i + j) % 3 * n + 1 elements to rank j
    cnt = [[((i + j) % 3) * n + 1 for j in range(p)] for i in range(p)]
    sends = [_rand(sum(cnt[i]), torch.float32, 800 + i) for i in range(p)]
    recvs = [torch.empty(sum(cnt[j][i] for j in range(p)), device="cuda") for i in range(p)]
    for i, c in enumerate(comms):
        sd = [sum(cnt[i][:j]) for j in range(p)]
        rc = [cnt[j][i] for j in range(p)]
        rd = [sum(rc[:j]) for j in range(p)]
        c.all_to_all_v(sends[i], cnt[i], sd, recvs[i], rc, rd)
    torch.cuda.synchronize()
    for i in range(p):
        off = 0
        for j in range(p):
            sd = sum(cnt[j][:i])
            assert torch.equal(recvs[i][off:off + cnt[j][i]], sends[j][sd:sd + cnt[j][i]])
            off += cnt[j][i]
    # same through the count-matrix form
    recvs2 = [torch.empty_like(r) for r in recvs]
    for i, c in enumerate(comms):
        c.all_to_all_vc(sends[i], cnt, recvs2[i])
    torch.cuda.synchronize()
    for a, b in zip(recvs, recvs2):
        assert torch.equal(a, b)


def test_v_variants(comms):
    p = len(comms)
    counts = [3 + 5 * r for r in range(p)]
    displs = [sum(counts[:r]) + r for r in range(p)]   # gaps between blocks
    total = displs[-1] + counts[-1]
    ins = [_rand(counts[r], torch.float32, 900 + r) for r in range(p)]
    outs = [torch.zeros(total, device="cuda") for _ in range(p)]
    for c, x, y in zip(comms, ins, outs):
        c.all_gather_v(x, y, counts, displs)
    torch.cuda.synchronize()
    for y in outs:
        for r in range(p):
            assert torch.equal(y[displs[r]:displs[r] + counts[r]], ins[r])
    sends = [_rand(total, torch.float32, 950 + r) for r in range(p)]
    recvs = [torch.empty(counts[r], device="cuda") for r in range(p)]
    for r, c in enumerate(comms):
        c.reduce_scatter_v(sends[r], recvs[r], counts, displs)
    torch.cuda.synchronize()
    ref = torch.stack([s.double() for s in sends]).sum(0)
    for r in range(p):
        torch.testing.assert_close(recvs[r].double(), ref[displs[r]:displs[r] + counts[r]], rtol=1e-5, atol=1e-5)


def test_batch_send_recv_ring_and_barrier(comms):
    p = len(comms)
    n = 300007
    sends = [_rand(n, torch.float32, 1000 + r) for r in range(p)]
    recvs = [torch.empty(n, device="cuda") for _ in range(p)]
    for rep in range(3):   # repeated: sequence numbers continue across launches
        for r, c in enumerate(comms):
            c.batch_send_recv([("send", sends[r], (r + 1) % p), ("recv", recvs[r], (r - 1) % p)])
        torch.cuda.synchronize()
        for r in range(p):
            assert torch.equal(recvs[r], sends[(r - 1) % p])
            recvs[r].zero_()
    for c in comms:
        c.barrier()
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS


def test_symmetric_memory_zero_copy(comms):
    p = len(comms)
    n = 1 << 18
    xs = [c.empty((n,), torch.bfloat16) for c in comms]
    ys = [c.empty((n,), torch.bfloat16) for c in comms]
    for r, x in enumerate(xs):
        x.copy_(_rand(n, torch.bfloat16, 1100 + r))
    for c, x, y in zip(comms, xs, ys):
        c.all_reduce(x, y)
    torch.cuda.synchronize()
    ref = torch.stack([x.double() for x in xs]).sum(0)
    for y in ys:
        torch.testing.assert_close(y.double(), ref, rtol=3e-2, atol=3e-2 * p)
    assert "TwoShot" in comms[0].last_algorithm() or "OneShot" in comms[0].last_algorithm() or "LL" in comms[0].last_algorithm()


def test_many_small_ops_back_to_back(comms):
    p = len(comms)
    xs = [_rand(256, torch.float32, 1200 + r) for r in range(p)]
    ref = torch.stack(xs).sum(0)
    ys = [torch.empty_like(x) for x in xs]
    for it in range(200):
        for c, x, y in zip(comms, xs, ys):
            c.all_reduce(x, y)
    torch.cuda.synchronize()
    for y in ys:
        torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)
    hits, misses, entries = comms[0].plan_cache_stats()
    assert hits >= 199


def test_unsignalled_wait_times_out_cleanly():
    """A wait that nothing satisfies must give up after the budget, report through
    the status block, and leave the CUDA context usable."""
    torch.cuda.set_device(0)
    cs = Communicator.emulated(2, hb.make_config(buffer_mib=8, exec_timeout_ms=300))
    from hccl_b200._lib import lib
    import ctypes

    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.HcclTestLaunchUnsignalledWait(cs[0].handle, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)) == 0
    t1.record()
    torch.cuda.synchronize()
    assert 250 <= t0.elapsed_time(t1) < 5000
    assert cs[0].async_error() == hb.Result.E_TIMEOUT
    assert cs[0].status() == hb.CommStatus.ERROR
    # the context still works
    x = torch.ones(10, device="cuda")
    assert float((x * 2).sum()) == 20.0
    with pytest.raises(hb.HcclError):
        cs[0].barrier()
    for c in cs:
        c.destroy()


def test_selector_on_device_communicator_and_resource_query():
    import ctypes

    from hccl_b200 import Cmd, DataType
    from hccl_b200._lib import HcclOpResource, lib

    torch.cuda.set_device(0)
    cs = Communicator.emulated(4, hb.make_config(buffer_mib=16))
    small = cs[0].explain(Cmd.ALLREDUCE, 256, DataType.FP32)
    big = cs[0].explain(Cmd.ALLREDUCE, 64 << 20, DataType.FP32)
    assert small.startswith("selected P2pAllReduceSoleMeshLL"), small
    assert big.startswith("selected P2pAllReduceSoleMeshPushTwoShot"), big      # ordinary buffers: slices pushed, no stage-in pass
    assert "NvlsAllReduceSoleMesh" not in big.split("\n")[0]          # no multicast on emulated ranks
    assert "Host" not in big                                           # host algorithms never compete on a device communicator
    r = HcclOpResource()
    # 64 Mi floats = 256 MiB through a 16 MiB slab: several launches, scratch bounded by the slab
    assert lib.HcclCalcOpResource(cs[0].handle, int(Cmd.ALLREDUCE), 64 << 20, int(DataType.FP32), 0, 0, ctypes.byref(r)) == 0
    assert r.algName.decode() == "P2pAllReduceSoleMeshPushTwoShot" and r.launches > 1 and r.streams == 1 and 0 < r.scratchBytes <= (16 << 20)
    assert lib.HcclCalcOpResource(cs[0].handle, int(Cmd.ALLREDUCE), 64 << 20, int(DataType.FP32), 0, 1, ctypes.byref(r)) == 0
    assert r.scratchBytes == 0            # symmetric buffers need no staging
    for c in cs:
        c.destroy()


def test_strict_determinism_repeats_bitwise():
    torch.cuda.set_device(0)
    p, n = 8, 300007
    ins = [(torch.randn(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(r)) * 10.0 ** (r - 4)).float() for r in range(p)]
    results = []
    for rep in range(2):
        cs = Communicator.emulated(p, hb.make_config(buffer_mib=16, deterministic=2))
        outs = [torch.empty_like(x) for x in ins]
        for c, x, y in zip(cs, ins, outs):
            c.all_reduce(x, y)
        torch.cuda.synchronize()
        assert "Nvls" not in cs[0].last_algorithm()
        for y in outs[1:]:
            assert torch.equal(y, outs[0])
        results.append(outs[0].clone())
        for c in cs:
            c.destroy()
    assert torch.equal(results[0], results[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int8, torch.int64])
@pytest.mark.parametrize("n", [1, 5, 1023, 4097, 30001])
def test_small_message_ll_forms(comms, dtype, n):
    """ReduceScatter, Broadcast and AlltoAll of small messages run as flag-in-data exchanges (no barrier); two rounds
    back to back so that both parities of the line slots are used."""
    p = len(comms)
    for rnd in range(2):
        ins = [_rand(n * p, dtype, 900 + 17 * rnd + r) for r in range(p)]
        outs = [torch.empty(n, device="cuda", dtype=dtype) for _ in range(p)]
        for c, x, y in zip(comms, ins, outs):
            c.reduce_scatter(x, y)
        es = ins[0].element_size()
        pair_ok = n * es <= 256 * 1024             # a pair's block has to fit one line slot
        if pair_ok and n * p * es <= 1024 * 1024:
            assert comms[0].last_algorithm() == "P2pReduceScatterSoleMeshLL"
        torch.cuda.synchronize()
        ref = torch.stack([x.double() for x in ins]).sum(0)
        for r, y in enumerate(outs):
            if dtype.is_floating_point:
                torch.testing.assert_close(y.double(), ref[r * n:(r + 1) * n], rtol=_tol(dtype), atol=_tol(dtype) * p)
            else:
                assert torch.equal(y.long(), ref[r * n:(r + 1) * n].long().to(dtype).long())

        a2a_out = [torch.empty(n * p, device="cuda", dtype=dtype) for _ in range(p)]
        for c, x, y in zip(comms, ins, a2a_out):
            c.all_to_all(x, y)
        if pair_ok and n * p * es <= 2 * 1024 * 1024:
            assert comms[0].last_algorithm() == "P2pAlltoAllSoleMeshLL"
        torch.cuda.synchronize()
        for r, y in enumerate(a2a_out):
            want = torch.cat([ins[q][r * n:(r + 1) * n] for q in range(p)])
            assert torch.equal(y.view(torch.uint8), want.view(torch.uint8))

        root = (rnd + 1) % p
        bufs = [x[:n].clone() for x in ins]
        want = bufs[root].clone()
        for c, b in zip(comms, bufs):
            c.broadcast(b, root)
        if n * es <= 64 * 1024:
            assert comms[0].last_algorithm() == "P2pBroadcastSoleMeshLL"
        torch.cuda.synchronize()
        for b in bufs:
            assert torch.equal(b.view(torch.uint8), want.view(torch.uint8))
    assert comms[0].async_error() == hb.Result.SUCCESS
