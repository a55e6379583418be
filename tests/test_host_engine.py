"""Host engine: N ranks as N host threads on host memory, running the
engine-agnostic algorithm templates (mesh one/two-shot, ring, RHD, NHR,
pairwise, sequence / parallel / order-preserved executors).  Numeric results
are compared with an fp64 oracle; the recorded primitive trace is verified for
deadlocks, bounds, memory conflicts and operator semantics."""
import os
import threading

import numpy as np
import pytest

import hccl_b200 as hb
from hccl_b200 import Communicator, ReduceOp
from hccl_b200._lib import lib


def run_ranks(comms, fn):
    """Runs fn(rank, comm) on one thread per rank; re-raises the first failure."""
    errs = [None] * len(comms)

    def body(r):
        try:
            fn(r, comms[r])
        except BaseException as e:  # noqa: BLE001
            errs[r] = e

    ts = [threading.Thread(target=body, args=(r,)) for r in range(len(comms))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for e in errs:
        if e is not None:
            raise e


@pytest.fixture
def algo_env():
    old = os.environ.get("HCCL_ALGO")
    yield
    if old is None:
        os.environ.pop("HCCL_ALGO", None)
    else:
        os.environ["HCCL_ALGO"] = old
    lib.HcclReloadEnvConfig()


def make(n, topo=None, algo=None, buffer_mib=64, deterministic=None):
    if algo is None:
        os.environ.pop("HCCL_ALGO", None)
    else:
        os.environ["HCCL_ALGO"] = algo
    lib.HcclReloadEnvConfig()
    return Communicator.host_sim(n, topo, hb.make_config(buffer_mib=buffer_mib, exec_timeout_ms=20000, deterministic=deterministic))


def destroy(comms):
    for c in comms:
        c.destroy()


ALGOS = {
    "ring": ("level0:NA;level1:ring", "Ring"),
    "rhd": ("level0:NA;level1:H-D_R", "RHD"),
    "nhr": ("level0:NA;level1:NHR", "NHR"),
    "mesh": ("level0:NA;level1:fullmesh", "Mesh"),
    "oneshot": ("level0:NA;level1:oneshot", "OneShot"),
}


def test_baseline_config_allreduce_fp32_8_ranks_ring_and_rhd(algo_env):
    """AllReduce(sum) fp32, 8 simulated ranks, 1,048,576 elements per rank, N(0,1)
    seeded by rank id, through the ring and the RHD templates; fp64 host sum, rel err <= 1e-6."""
    n, count = 8, 1 << 20
    ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
    ref = np.sum(np.stack(ins).astype(np.float64), axis=0)
    for key in ("ring", "rhd"):
        comms = make(n, algo=ALGOS[key][0])
        outs = [np.empty(count, np.float32) for _ in range(n)]
        run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r], ReduceOp.SUM))
        assert ALGOS[key][1] in comms[0].last_algorithm()
        for o in outs:
            rel = np.abs(o.astype(np.float64) - ref).max() / np.abs(ref).max()
            assert rel <= 1e-6, (key, rel)
        destroy(comms)


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 7, 8, 16])
@pytest.mark.parametrize("key", list(ALGOS))
def test_allreduce_algorithms_and_rank_counts(algo_env, n, key):
    comms = make(n, algo=ALGOS[key][0])
    for count in (1, 5, 1000, 4097):
        ins = [np.random.default_rng(100 + r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        report = comms[0].trace_verify()
        assert report.startswith("OK"), report
        ref = np.sum(np.stack(ins).astype(np.float64), axis=0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-6 * n)
    if n > 1:
        assert ALGOS[key][1] in comms[0].last_algorithm(), comms[0].last_algorithm()
    destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 5, 8, 12])
@pytest.mark.parametrize("key", ["ring", "rhd", "nhr", "mesh"])
def test_reduce_scatter_all_gather(algo_env, n, key):
    comms = make(n, algo=ALGOS[key][0])
    for count in (1, 33, 2049):
        ins = [np.random.default_rng(7 + r).standard_normal(count * n).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.reduce_scatter(ins[r], outs[r]))
        assert comms[0].trace_verify().startswith("OK")
        ref = np.sum(np.stack(ins).astype(np.float64), axis=0)
        for r, o in enumerate(outs):
            np.testing.assert_allclose(o, ref[r * count:(r + 1) * count], rtol=2e-6, atol=2e-6 * n)
        gin = [np.random.default_rng(50 + r).integers(-100, 100, count).astype(np.int32) for r in range(n)]
        gout = [np.zeros(count * n, np.int32) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.all_gather(gin[r], gout[r]))
        assert comms[0].trace_verify().startswith("OK")
        for o in gout:
            assert np.array_equal(o, np.concatenate(gin))
    destroy(comms)


@pytest.mark.parametrize("dtype", [np.int8, np.int16, np.int32, np.int64, np.uint64, np.float16, np.float32, np.float64])
@pytest.mark.parametrize("op", [ReduceOp.SUM, ReduceOp.MAX, ReduceOp.MIN, ReduceOp.PROD])
def test_dtype_op_matrix(algo_env, dtype, op):
    if op == ReduceOp.PROD and dtype in (np.int16,):
        pytest.skip("prod is not defined for int16")
    n, count = 4, 257
    comms = make(n)
    rng = np.random.default_rng(3)
    if np.issubdtype(dtype, np.floating):
        ins = [(rng.random(count) + 0.5).astype(dtype) for _ in range(n)]
    else:
        ins = [rng.integers(1, 3, count).astype(dtype) for _ in range(n)]
    outs = [np.zeros(count, dtype) for _ in range(n)]
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r], op))
    st = np.stack(ins).astype(np.float64)
    ref = {ReduceOp.SUM: st.sum(0), ReduceOp.MAX: st.max(0), ReduceOp.MIN: st.min(0), ReduceOp.PROD: st.prod(0)}[op]
    tol = 2e-2 if dtype == np.float16 else 1e-6
    for o in outs:
        np.testing.assert_allclose(o.astype(np.float64), ref, rtol=tol, atol=tol)
    destroy(comms)


def test_rooted_and_alltoall_ops(algo_env):
    n, count = 6, 301
    for algo in (None, "level0:NA;level1:NHR", "level0:NA;level1:ring", "alltoall=level0:NA;level1:pairwise"):
        comms = make(n, algo=algo)
        root = 2
        bufs = [np.full(count, r, np.float32) for r in range(n)]
        run_ranks(comms, lambda r, c: c.broadcast(bufs[r], root))
        for b in bufs:
            assert np.all(b == root)
        ins = [np.random.default_rng(r).standard_normal(count).astype(np.float64) for r in range(n)]
        out = np.zeros(count, np.float64)
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.reduce(ins[r], out if r == root else None, root))
        assert comms[0].trace_verify().startswith("OK")
        np.testing.assert_allclose(out, np.sum(np.stack(ins), 0), rtol=1e-12)
        src = np.arange(count * n, dtype=np.int32)
        outs = [np.zeros(count, np.int32) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.scatter(src if r == root else None, outs[r], root))
        assert comms[0].trace_verify().startswith("OK")
        for r, o in enumerate(outs):
            assert np.array_equal(o, src[r * count:(r + 1) * count])
        a2a_in = [np.arange(count * n, dtype=np.int64) + 1000000 * r for r in range(n)]
        a2a_out = [np.zeros(count * n, np.int64) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.all_to_all(a2a_in[r], a2a_out[r]))
        assert comms[0].trace_verify().startswith("OK")
        for r in range(n):
            for q in range(n):
                assert np.array_equal(a2a_out[r][q * count:(q + 1) * count], a2a_in[q][r * count:(r + 1) * count])
        if algo and "pairwise" in algo:
            assert "Pairwise" in comms[0].last_algorithm()
        # variable counts through V and VC
        cnt = [[(i * 3 + j) % 4 + 1 for j in range(n)] for i in range(n)]
        sends = [np.arange(sum(cnt[i]), dtype=np.float32) + 100 * i for i in range(n)]
        recvs = [np.zeros(sum(cnt[j][i] for j in range(n)), np.float32) for i in range(n)]

        def a2av(i, c):
            sd = [sum(cnt[i][:j]) for j in range(n)]
            rc = [cnt[j][i] for j in range(n)]
            rd = [sum(rc[:j]) for j in range(n)]
            c.all_to_all_v(sends[i], cnt[i], sd, recvs[i], rc, rd)

        run_ranks(comms, a2av)
        recvs2 = [np.zeros_like(x) for x in recvs]
        run_ranks(comms, lambda i, c: c.all_to_all_vc(sends[i], cnt, recvs2[i]))
        for i in range(n):
            off = 0
            for j in range(n):
                sd = sum(cnt[j][:i])
                assert np.array_equal(recvs[i][off:off + cnt[j][i]], sends[j][sd:sd + cnt[j][i]])
                off += cnt[j][i]
            assert np.array_equal(recvs[i], recvs2[i])
        # send / recv ring and barrier
        got = [np.zeros(17, np.int32) for _ in range(n)]
        run_ranks(comms, lambda r, c: c.batch_send_recv([("send", np.full(17, r, np.int32), (r + 1) % n), ("recv", got[r], (r - 1) % n)]))
        for r in range(n):
            assert np.all(got[r] == (r - 1) % n)
        run_ranks(comms, lambda r, c: c.barrier())
        destroy(comms)


def test_serial_windowed_all_to_all(algo_env):
    """AlltoAll / AlltoAllV one peer at a time (rank ^ step) through the staging buffer in windows of half of it
    (reference: ins_v2_all_to_all_v_serial_sole_executor.cc:113-171): with a 1 MiB buffer the larger pairs take up to
    four windows, so both halves are reused; rank counts that are and are not powers of two; a pair that sends
    nothing one way; the trace verifier sees no race on the staging halves and no deadlock."""
    for n in (2, 5, 8):
        comms = make(n, algo="alltoall=level0:NA;level1:serial", buffer_mib=1)
        count = 70001                                            # x 8 bytes: 547 KiB per pair = two windows of 512 KiB
        a2a_in = [np.arange(count * n, dtype=np.int64) + 10000000 * r for r in range(n)]
        a2a_out = [np.zeros(count * n, np.int64) for _ in range(n)]
        comms[0].trace_begin()
        run_ranks(comms, lambda r, c: c.all_to_all(a2a_in[r], a2a_out[r]))
        assert comms[0].trace_verify().startswith("OK"), comms[0].trace_verify()
        assert "SerialSoleMesh" in comms[0].last_algorithm()
        for r in range(n):
            for q in range(n):
                assert np.array_equal(a2a_out[r][q * count:(q + 1) * count], a2a_in[q][r * count:(r + 1) * count])
        # uneven counts: up to ~1.9 MiB one way (four windows) and nothing the other way for some pairs
        cnt = [[0 if (i + 2 * j) % 5 == 1 else ((i * 7 + j * 13) % 9) * 53003 + 17 for j in range(n)] for i in range(n)]
        sends = [np.arange(sum(cnt[i]), dtype=np.float32) + 0.5 * i for i in range(n)]
        recvs = [np.zeros(sum(cnt[j][i] for j in range(n)), np.float32) for i in range(n)]

        def a2av(i, c):
            sd = [sum(cnt[i][:j]) for j in range(n)]
            rc = [cnt[j][i] for j in range(n)]
            rd = [sum(rc[:j]) for j in range(n)]
            c.all_to_all_v(sends[i], cnt[i], sd, recvs[i], rc, rd)

        comms[0].trace_begin()
        run_ranks(comms, a2av)
        assert comms[0].trace_verify().startswith("OK"), comms[0].trace_verify()
        assert "SerialSoleMesh" in comms[0].last_algorithm()
        recvs2 = [np.zeros_like(x) for x in recvs]
        run_ranks(comms, lambda i, c: c.all_to_all_vc(sends[i], cnt, recvs2[i]))
        for i in range(n):
            off = 0
            for j in range(n):
                sd = sum(cnt[j][:i])
                assert np.array_equal(recvs[i][off:off + cnt[j][i]], sends[j][sd:sd + cnt[j][i]])
                off += cnt[j][i]
            assert np.array_equal(recvs[i], recvs2[i])
        destroy(comms)


def test_v_variants_host(algo_env):
    n = 5
    comms = make(n)
    counts = [2 + 3 * r for r in range(n)]
    displs = [sum(counts[:r]) + 2 * r for r in range(n)]
    total = displs[-1] + counts[-1]
    ins = [np.full(counts[r], r + 1, np.float32) for r in range(n)]
    outs = [np.zeros(total, np.float32) for _ in range(n)]
    run_ranks(comms, lambda r, c: c.all_gather_v(ins[r], outs[r], counts, displs))
    for o in outs:
        for r in range(n):
            assert np.all(o[displs[r]:displs[r] + counts[r]] == r + 1)
    sends = [np.random.default_rng(r).standard_normal(total).astype(np.float32) for r in range(n)]
    recvs = [np.zeros(counts[r], np.float32) for r in range(n)]
    run_ranks(comms, lambda r, c: c.reduce_scatter_v(sends[r], recvs[r], counts, displs))
    ref = np.sum(np.stack(sends).astype(np.float64), 0)
    for r in range(n):
        np.testing.assert_allclose(recvs[r], ref[displs[r]:displs[r] + counts[r]], rtol=1e-5, atol=1e-5)
    destroy(comms)


@pytest.mark.parametrize("topo,n", [("[[[0,1,2,3],[4,5,6,7]]]", 8), ("[[[0,1],[2,3],[4,5]]]", 6), ("[[[0,1],[2,3]],[[4,5],[6,7]]]", 8)])
@pytest.mark.parametrize("algo", ["level0:NA;level1:NHR", "level0:NA;level1:ring", "level0:NA;level1:H-D_R", "level0:NA;level1:pipeline"])
def test_hierarchical_executors(algo_env, topo, n, algo):
    comms = make(n, topo=topo, algo=algo)
    count = 1537
    ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
    outs = [np.zeros(count, np.float32) for _ in range(n)]
    comms[0].trace_begin()
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
    rep = comms[0].trace_verify()
    assert rep.startswith("OK"), rep
    ref = np.sum(np.stack(ins).astype(np.float64), 0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
    name = comms[0].last_algorithm()
    assert "Sequence" in name or "Parallel" in name, name
    # hierarchical ReduceScatter / AllGather
    rs_in = [np.random.default_rng(30 + r).standard_normal(64 * n).astype(np.float32) for r in range(n)]
    rs_out = [np.zeros(64, np.float32) for _ in range(n)]
    comms[0].trace_begin()
    run_ranks(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
    assert comms[0].trace_verify().startswith("OK")
    assert ("Parallel" if "pipeline" in algo else "Sequence") in comms[0].last_algorithm(), comms[0].last_algorithm()
    ref = np.sum(np.stack(rs_in).astype(np.float64), 0)
    for r in range(n):
        np.testing.assert_allclose(rs_out[r], ref[r * 64:(r + 1) * 64], rtol=2e-6, atol=2e-5)
    ag_out = [np.zeros(64 * n, np.float32) for _ in range(n)]
    comms[0].trace_begin()
    run_ranks(comms, lambda r, c: c.all_gather(rs_out[r], ag_out[r]))
    assert comms[0].trace_verify().startswith("OK")
    assert ("Parallel" if "pipeline" in algo else "Sequence") in comms[0].last_algorithm(), comms[0].last_algorithm()
    for o in ag_out:
        np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
    destroy(comms)


def test_strict_determinism_is_bitwise_and_order_preserved(algo_env):
    n, count = 7, 10007
    ins = [(np.random.default_rng(r).standard_normal(count) * 10.0 ** np.random.default_rng(r + 99).integers(-3, 4, count)).astype(np.float32) for r in range(n)]
    results = []
    for rep in range(2):
        comms = make(n, deterministic=2)
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        for o in outs[1:]:
            assert o.tobytes() == outs[0].tobytes()
        results.append(outs[0].tobytes())
        destroy(comms)
    assert results[0] == results[1]


def test_chunk_loop_when_message_exceeds_scratch(algo_env):
    n, count = 4, 700001          # 2.8 MB per rank through a 1 MiB scratch buffer
    comms = make(n, buffer_mib=1)
    ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
    outs = [np.zeros(count, np.float32) for _ in range(n)]
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
    ref = np.sum(np.stack(ins).astype(np.float64), 0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
    destroy(comms)


def test_strict_order_is_batch_invariant(algo_env):
    """The ordered reduction gives the same bits whether a message goes through in one piece or in chunks, and whether
    an element is reduced alone or as part of a longer vector (the property the reference's batch-invariant
    ReduceScatter / AllReduce variants are built for)."""
    n, count = 5, 300001
    ins = [(np.random.default_rng(r).standard_normal(count) * 10.0 ** np.random.default_rng(r + 7).integers(-4, 5, count)).astype(np.float32) for r in range(n)]

    def run(buffer_mib, lo, hi):
        comms = make(n, buffer_mib=buffer_mib, deterministic=2)
        outs = [np.zeros(hi - lo, np.float32) for _ in range(n)]
        run_ranks(comms, lambda r, c: c.all_reduce(ins[r][lo:hi].copy(), outs[r]))
        destroy(comms)
        return outs[0]

    whole = run(64, 0, count)
    chunked = run(1, 0, count)                  # 1.2 MB per rank through a 1 MiB buffer: several loops
    assert whole.tobytes() == chunked.tobytes()
    part = run(64, 1000, 1777)                  # the same elements as a short message
    assert part.tobytes() == whole[1000:1777].tobytes()
    # ReduceScatter of the same data agrees bit for bit with the matching block of the AllReduce
    m = count // n
    comms = make(n, deterministic=2)
    rs_out = [np.zeros(m, np.float32) for _ in range(n)]
    run_ranks(comms, lambda r, c: c.reduce_scatter(ins[r][:m * n].copy(), rs_out[r]))
    destroy(comms)
    for r in range(n):
        assert rs_out[r].tobytes() == whole[r * m:(r + 1) * m].tobytes()


def test_stress_mixed_operators_back_to_back(algo_env):
    """Three hundred operators of random kind, size and root in a row on one communicator: notify counters, scratch
    reuse and the rendezvous survive any succession, and every result is right."""
    n = 4
    rng = np.random.default_rng(123)
    plan = [(rng.choice(["ar", "ag", "rs", "bc", "a2a", "red", "sc", "bar"]), int(rng.integers(1, 3000)), int(rng.integers(0, n))) for _ in range(300)]
    for algo in (None, "level0:NA;level1:NHR"):
        comms = make(n, algo=algo, buffer_mib=4)
        fails = []

        def body(r, c):
            for i, (kind, count, root) in enumerate(plan):
                base = np.arange(count, dtype=np.int64) * (r + 1) + i
                if kind == "ar":
                    out = np.zeros(count, np.int64)
                    c.all_reduce(base, out)
                    want = sum(np.arange(count, dtype=np.int64) * (q + 1) + i for q in range(n))
                elif kind == "ag":
                    out = np.zeros(count * n, np.int64)
                    c.all_gather(base, out)
                    want = np.concatenate([np.arange(count, dtype=np.int64) * (q + 1) + i for q in range(n)])
                elif kind == "rs":
                    src = np.arange(count * n, dtype=np.int64) * (r + 1) + i
                    out = np.zeros(count, np.int64)
                    c.reduce_scatter(src, out)
                    want = sum(np.arange(count * n, dtype=np.int64) * (q + 1) + i for q in range(n))[r * count:(r + 1) * count]
                elif kind == "bc":
                    out = base.copy()
                    c.broadcast(out, root)
                    want = np.arange(count, dtype=np.int64) * (root + 1) + i
                elif kind == "a2a":
                    src = np.arange(count * n, dtype=np.int64) * (r + 1) + i
                    out = np.zeros(count * n, np.int64)
                    c.all_to_all(src, out)
                    want = np.concatenate([(np.arange(count * n, dtype=np.int64) * (q + 1) + i)[r * count:(r + 1) * count] for q in range(n)])
                elif kind == "red":
                    out = np.zeros(count, np.int64)
                    c.reduce(base, out if r == root else None, root)
                    want = sum(np.arange(count, dtype=np.int64) * (q + 1) + i for q in range(n)) if r == root else out
                elif kind == "sc":
                    src = np.arange(count * n, dtype=np.int64) + i
                    out = np.zeros(count, np.int64)
                    c.scatter(src if r == root else None, out, root)
                    want = src[r * count:(r + 1) * count]
                else:
                    c.barrier()
                    continue
                if not np.array_equal(out, want):
                    fails.append((i, kind, count, root, r))

        run_ranks(comms, body)
        assert not fails, fails[:5]
        destroy(comms)
