"""Host engine: Concurrent, Pipeline, Nonuniform Bruck, hierarchical AlltoAll,
two-level Sequence forms of the rooted operators, and the tree-interpreting
executor.  Every case checks the numbers against a NumPy oracle and the
recorded trace against the verifier (deadlock, bounds, memory conflicts,
operator semantics)."""
import ctypes
import os

import numpy as np
import pytest

import hccl_b200 as hb
from hccl_b200._lib import lib

from test_host_engine import algo_env, destroy, make, run_ranks  # noqa: F401

TWO_BY_FOUR = "[[[0,1,2,3],[4,5,6,7]]]"
THREE_BY_TWO = "[[[0,1],[2,3],[4,5]]]"
TWO_PODS = "[[[0,1],[2,3]],[[4,5],[6,7]]]"


def step_table(kind, p, rank, arg=None):
    buf = ctypes.create_string_buffer(1 << 16)
    rc = lib.HcclDebugStepTable(kind.encode(), p, rank, arg.encode() if arg else None, buf, len(buf))
    assert rc == 0, rc
    return buf.value.decode()


def verified(comms, fn):
    comms[0].trace_begin()
    run_ranks(comms, fn)
    rep = comms[0].trace_verify()
    assert rep.startswith("OK"), rep


# ---------------------------------------------------------------- step tables
@pytest.mark.parametrize("p", [2, 3, 5, 6, 8, 13])
def test_bruck_allgather_table_covers_every_block_once(p):
    have = [{r} for r in range(p)]
    steps = [step_table("bruck_ag", p, r).strip().splitlines() for r in range(p)]
    n_steps = (p - 1).bit_length()
    assert all(len(s) == n_steps for s in steps)
    for s in range(n_steps):
        sent = []
        for r in range(p):
            f = steps[r][s].split()
            to, frm, first_send, first_recv, n = int(f[1]), int(f[3]), int(f[5]), int(f[7]), int(f[9])
            assert to == (r - (1 << s)) % p and frm == (r + (1 << s)) % p
            assert first_send == r and first_recv == frm and n == min(1 << s, p - (1 << s))
            blocks = {(first_send + k) % p for k in range(n)}
            assert blocks <= have[r]
            sent.append((to, blocks))
        for to, blocks in sent:
            assert not (blocks & have[to])       # nothing is sent twice
            have[to] |= blocks
    assert all(h == set(range(p)) for h in have)


@pytest.mark.parametrize("p", [2, 3, 5, 8, 11])
def test_binomial_scatter_table_delivers_every_block(p):
    holds = {0: set(range(p))}
    tables = [step_table("nb_scatter", p, v).strip().splitlines() for v in range(p)]
    for s in range(len(tables[0])):
        for v in range(p):
            f = tables[v][s].split()
            if f[0] != "send":
                continue
            peer, first, n = int(f[2]), int(f[4]), int(f[6])
            blocks = set(range(first, first + n))
            assert blocks <= holds[v]
            g = tables[peer][s].split()
            assert g[0] == "recv" and int(g[2]) == v and int(g[4]) == first and int(g[6]) == n
            holds[peer] = blocks
            holds[v] -= blocks
    assert all(v in holds[v] for v in range(p))


def test_bandwidth_split_and_pipeline_schedule():
    assert step_table("bw_split", 0, 0, "3000,56,112,32").strip() == "992"      # a third, cut down to 32 elements
    assert step_table("bw_split", 0, 0, "40,56,112,32").strip() == "0"          # part A below one unit: B takes all
    assert step_table("bw_split", 0, 0, "100,1,0,1").strip() == "100"
    assert step_table("bw_split", 0, 0, "64,1,1,1").strip() == "32"
    slots = [tuple(int(x) for x in l.split()[1::2]) for l in step_table("pipeline", 3, 4).strip().splitlines()]
    assert len(slots) == 12 and len(set(slots)) == 12
    for t, stage, step in slots:
        assert t == stage + step
    # a stage of a step never precedes the stage before it
    pos = {(stage, step): i for i, (t, stage, step) in enumerate(slots)}
    for step in range(4):
        assert pos[(0, step)] < pos[(1, step)] < pos[(2, step)]


def test_tree_text_is_parsed_and_rejected():
    ok = step_table("parse_tree", 0, 0, " par( seq(mesh, nhr) , rev(seq(NHR,mesh)), 1:3 ) ")
    assert ok.strip() == "par(seq(mesh,nhr),rev(seq(nhr,mesh)),1:3) queues 2 levels 2"
    assert step_table("parse_tree", 0, 0, "seq(mesh,ring,nb)").strip() == "seq(mesh,ring,nb) queues 1 levels 3"
    for bad in ("", "seq(mesh)", "par(mesh)", "seq(seq(mesh,nhr),ring)", "butterfly", "seq(mesh,nhr", "par(mesh,nhr,0:0)", "mesh)"):
        assert step_table("parse_tree", 0, 0, bad).startswith("error:"), bad


# ---------------------------------------------------------------- executors
@pytest.mark.parametrize("n", [2, 3, 5, 8])
def test_concurrent_executors(algo_env, n):
    comms = make(n, algo="level0:NA;level1:concurrent")
    for count in (1, 31, 4099):
        ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert "Concurrent" in comms[0].last_algorithm()
        ref = np.sum(np.stack(ins).astype(np.float64), 0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
        rs_in = [np.random.default_rng(9 + r).standard_normal(count * n).astype(np.float32) for r in range(n)]
        rs_out = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
        assert "Concurrent" in comms[0].last_algorithm()
        ref = np.sum(np.stack(rs_in).astype(np.float64), 0)
        for r in range(n):
            np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=2e-6, atol=2e-5)
        ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int32) for r in range(n)]
        ag_out = [np.zeros(count * n, np.int32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
        assert "Concurrent" in comms[0].last_algorithm()
        for o in ag_out:
            assert np.array_equal(o, np.concatenate(ag_in))
        a2a_in = [np.arange(count * n, dtype=np.int64) + 1000000 * r for r in range(n)]
        a2a_out = [np.zeros(count * n, np.int64) for _ in range(n)]
        verified(comms, lambda r, c: c.all_to_all(a2a_in[r], a2a_out[r]))
        assert comms[0].last_algorithm() == "HostAlltoAllConcurrentMeshMesh", comms[0].last_algorithm()
        for r in range(n):
            for q in range(n):
                assert np.array_equal(a2a_out[r][q * count:(q + 1) * count], a2a_in[q][r * count:(r + 1) * count])
        cnt = [[(i * 3 + j * 5 + count) % 7 for j in range(n)] for i in range(n)]          # zeros included
        sends = [np.arange(sum(cnt[i]), dtype=np.float32) + 100 * i for i in range(n)]
        recvs = [np.zeros(sum(cnt[j][i] for j in range(n)), np.float32) for i in range(n)]

        def a2av(i, c):
            sd = [sum(cnt[i][:j]) for j in range(n)]
            rc = [cnt[j][i] for j in range(n)]
            rd = [sum(rc[:j]) for j in range(n)]
            c.all_to_all_v(sends[i], cnt[i], sd, recvs[i], rc, rd)

        verified(comms, a2av)
        assert comms[0].last_algorithm() == "HostAlltoAllVConcurrentMeshMesh", comms[0].last_algorithm()
        recvs2 = [np.zeros_like(v) for v in recvs]
        verified(comms, lambda i, c: c.all_to_all_vc(sends[i], cnt, recvs2[i]))
        for i in range(n):
            off = 0
            for j in range(n):
                sd = sum(cnt[j][:i])
                assert np.array_equal(recvs[i][off:off + cnt[j][i]], sends[j][sd:sd + cnt[j][i]])
                off += cnt[j][i]
            assert np.array_equal(recvs[i], recvs2[i])
        for root in (0, n - 1):
            bufs = [np.full(count, 100 + r, np.int16) for r in range(n)]
            verified(comms, lambda r, c: c.broadcast(bufs[r], root))
            assert comms[0].last_algorithm() == "HostBroadcastConcurrentMeshNHR", comms[0].last_algorithm()
            assert all(np.all(b == 100 + root) for b in bufs)
            sc_in = np.random.default_rng(90 + root).integers(-1000, 1000, count * n).astype(np.int32)
            sc_out = [np.zeros(count, np.int32) for _ in range(n)]
            verified(comms, lambda r, c: c.scatter(sc_in if r == root else None, sc_out[r], root))
            assert comms[0].last_algorithm() == "HostScatterConcurrentMeshMesh", comms[0].last_algorithm()
            for r in range(n):
                assert np.array_equal(sc_out[r], sc_in[r * count:(r + 1) * count])
            red_in = [np.random.default_rng(70 + r).standard_normal(count) for r in range(n)]
            red_out = np.zeros(count, np.float64)
            verified(comms, lambda r, c: c.reduce(red_in[r], red_out if r == root else None, root))
            assert comms[0].last_algorithm() == "HostReduceConcurrentMeshNHR", comms[0].last_algorithm()
            np.testing.assert_allclose(red_out, np.sum(np.stack(red_in), 0), rtol=1e-12, atol=1e-13)
    destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 5, 8])
@pytest.mark.parametrize("algo,name", [("allreduce=level0:2die", "HostAllReduceSequence2DieMeshMesh"), ("allreduce=level0:meshconcur", "HostAllReduceSoleMeshConcur")])
def test_all_reduce_over_two_link_sets(algo_env, n, algo, name):
    """Two-shot AllReduce whose peers (two-die sequence) or whose data (mesh over both link sets at once) are divided
    between two queues; odd rank counts leave the halves unequal; the verifier sees no two queues fold into one place."""
    comms = make(n, algo=algo)
    for count in (1, 7, 4099, 100003):
        ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert comms[0].last_algorithm() == name, comms[0].last_algorithm()
        ref = np.sum(np.stack(ins).astype(np.float64), 0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
    destroy(comms)


def test_concurrent_split_follows_the_ratio_variable(algo_env):
    os.environ["HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO"] = "1,0"
    try:
        n, count = 4, 1000
        comms = make(n, algo="level0:NA;level1:concurrent")
        ins = [np.full(count, r + 1, np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert all(np.all(o == 10) for o in outs)
        destroy(comms)
    finally:
        os.environ.pop("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO")
        lib.HcclReloadEnvConfig()


@pytest.mark.parametrize("topo,n", [(TWO_BY_FOUR, 8), (THREE_BY_TWO, 6)])
def test_pipeline_executors(algo_env, topo, n):
    comms = make(n, topo=topo, algo="level0:NA;level1:omnipipe")
    for count in (3, 640, 20011):
        ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert "Pipeline" in comms[0].last_algorithm()
        ref = np.sum(np.stack(ins).astype(np.float64), 0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
        ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int64) for r in range(n)]
        ag_out = [np.zeros(count * n, np.int64) for _ in range(n)]
        verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
        assert "Pipeline" in comms[0].last_algorithm()
        for o in ag_out:
            assert np.array_equal(o, np.concatenate(ag_in))
        rs_in = [np.random.default_rng(40 + r).standard_normal(count * n) for r in range(n)]
        rs_out = [np.zeros(count, np.float64) for _ in range(n)]
        verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
        assert "Pipeline" in comms[0].last_algorithm()
        ref = np.sum(np.stack(rs_in), 0)
        for r in range(n):
            np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=1e-12, atol=1e-13)
        for root in (0, n - 1):
            bufs = [np.full(count, 100 + r, np.int16) for r in range(n)]
            verified(comms, lambda r, c: c.broadcast(bufs[r], root))
            assert "Pipeline" in comms[0].last_algorithm()
            assert all(np.all(b == 100 + root) for b in bufs)
            counts = [(count * (r + 1)) // n + (r % 2) for r in range(n)]          # AllGatherV: uneven blocks with gaps
            displs = [sum(counts[:r]) + 3 * r for r in range(n)]
            agv_in = [np.random.default_rng(50 + r).integers(-99, 99, counts[r]).astype(np.int16) for r in range(n)]
            agv_out = [np.full(displs[-1] + counts[-1], -777, np.int16) for _ in range(n)]
            verified(comms, lambda r, c: c.all_gather_v(agv_in[r], agv_out[r], counts, displs))
            assert comms[0].last_algorithm() == "HostAllGatherVPipelineMeshMesh", comms[0].last_algorithm()
            for o in agv_out:
                for r in range(n):
                    assert np.array_equal(o[displs[r]:displs[r] + counts[r]], agv_in[r])
                    assert np.all(o[displs[r] + counts[r]:displs[r] + counts[r] + 3][:3 if r < n - 1 else 0] == -777)
            red_in = [np.random.default_rng(70 + r).standard_normal(count) for r in range(n)]
            red_out = np.zeros(count, np.float64)
            verified(comms, lambda r, c: c.reduce(red_in[r], red_out if r == root else None, root))
            assert comms[0].last_algorithm() == "HostReducePipelineMeshNHR", comms[0].last_algorithm()
            np.testing.assert_allclose(red_out, np.sum(np.stack(red_in), 0), rtol=1e-12, atol=1e-13)
            sc_in = np.random.default_rng(90 + root).integers(-1000, 1000, count * n).astype(np.int32)
            sc_out = [np.zeros(count, np.int32) for _ in range(n)]
            verified(comms, lambda r, c: c.scatter(sc_in if r == root else None, sc_out[r], root))
            assert comms[0].last_algorithm() == "HostScatterPipelineMeshMesh", comms[0].last_algorithm()
            for r in range(n):
                assert np.array_equal(sc_out[r], sc_in[r * count:(r + 1) * count])
    destroy(comms)


@pytest.mark.parametrize("ratio", [None, "1,0", "0,1", "3,1"])
def test_parallel_all_gather_and_reduce_scatter(algo_env, ratio):
    """Parallel executors: part A of every block goes server first, then column; part B column first, then server, on
    a second queue (reference: CalcParallelDataSplitRatio, template_utils.h:809-826).  Every split ratio, parts that are
    empty included, gives the same values; the trace verifier sees no race between the two parts."""
    if ratio:
        os.environ["HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO"] = ratio
    try:
        for topo, n in ((TWO_BY_FOUR, 8), (THREE_BY_TWO, 6)):
            comms = make(n, topo=topo, algo="level0:NA;level1:pipeline")
            for count in (1, 64, 20011):
                ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int32) for r in range(n)]
                ag_out = [np.zeros(count * n, np.int32) for _ in range(n)]
                verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
                assert comms[0].last_algorithm() == "HostAllGatherParallelMeshMesh", comms[0].last_algorithm()
                for o in ag_out:
                    assert np.array_equal(o, np.concatenate(ag_in))
                rs_in = [np.random.default_rng(40 + r).standard_normal(count * n) for r in range(n)]
                rs_out = [np.zeros(count, np.float64) for _ in range(n)]
                verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
                assert comms[0].last_algorithm() == "HostReduceScatterParallelMeshMesh", comms[0].last_algorithm()
                ref = np.sum(np.stack(rs_in), 0)
                for r in range(n):
                    np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=1e-12, atol=1e-13)
                assert all(np.array_equal(rs_in[r], np.random.default_rng(40 + r).standard_normal(count * n)) for r in range(n))   # inputs intact
                for root in (0, n // 2, n - 1):                  # the rooted operators: the root in the first, a middle and the last server
                    bufs = [np.full(count, 100 + r, np.int16) for r in range(n)]
                    verified(comms, lambda r, c: c.broadcast(bufs[r], root))
                    assert comms[0].last_algorithm() == "HostBroadcastParallelMeshMesh", comms[0].last_algorithm()
                    assert all(np.all(b == 100 + root) for b in bufs)
                    red_in = [np.random.default_rng(70 + r).standard_normal(count) for r in range(n)]
                    red_out = np.zeros(count, np.float64)
                    verified(comms, lambda r, c: c.reduce(red_in[r], red_out if r == root else None, root))
                    assert comms[0].last_algorithm() == "HostReduceParallelMeshNHR", comms[0].last_algorithm()
                    np.testing.assert_allclose(red_out, np.sum(np.stack(red_in), 0), rtol=1e-12, atol=1e-13)
                    sc_in = np.random.default_rng(90 + root).integers(-1000, 1000, count * n).astype(np.int32)
                    sc_out = [np.zeros(count, np.int32) for _ in range(n)]
                    verified(comms, lambda r, c: c.scatter(sc_in if r == root else None, sc_out[r], root))
                    assert comms[0].last_algorithm() == "HostScatterParallelMeshMesh", comms[0].last_algorithm()
                    for r in range(n):
                        assert np.array_equal(sc_out[r], sc_in[r * count:(r + 1) * count])
            destroy(comms)
    finally:
        os.environ.pop("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", None)
        lib.HcclReloadEnvConfig()


@pytest.mark.parametrize("topo,n", [(TWO_PODS, 8), ("[[[0,1,2],[3,4,5]],[[6,7,8],[9,10,11]],[[12,13,14],[15,16,17]]]", 18)])
def test_three_level_pipeline_all_reduce(algo_env, topo, n):
    """Servers, pods and the level above them: five pipelined stages (mesh ReduceScatter, NHR ReduceScatter, NHR
    AllReduce, NHR AllGather, mesh AllGather), checked against the fp64 sum and by the trace verifier."""
    comms = make(n, topo=topo, algo="level0:NA;level1:omnipipe;level2:omnipipe")
    for count in (1, 5, 977, 30011):
        ins = [np.random.default_rng(100 + r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert comms[0].last_algorithm() == "HostAllReducePipelineMeshNHRNHR", comms[0].last_algorithm()
        ref = np.sum(np.stack(ins).astype(np.float64), 0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=3e-6, atol=3e-5)
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
        ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int64) for r in range(n)]
        ag_out = [np.zeros(count * n, np.int64) for _ in range(n)]
        verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
        assert comms[0].last_algorithm() == "HostAllGatherPipelineMeshMeshMesh", comms[0].last_algorithm()
        for o in ag_out:
            assert np.array_equal(o, np.concatenate(ag_in))
        rs_in = [np.random.default_rng(40 + r).standard_normal(count * n) for r in range(n)]
        rs_out = [np.zeros(count, np.float64) for _ in range(n)]
        verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
        assert comms[0].last_algorithm() == "HostReduceScatterPipelineMeshMeshMesh", comms[0].last_algorithm()
        ref = np.sum(np.stack(rs_in), 0)
        for r in range(n):
            np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=1e-12, atol=1e-13)
    destroy(comms)


@pytest.mark.parametrize("topo,n", [(TWO_PODS, 8), ("[[[0,1,2],[3,4,5]],[[6,7,8],[9,10,11]],[[12,13,14],[15,16,17]]]", 18)])
def test_three_level_sequence_all_gather_and_reduce_scatter(algo_env, topo, n):
    """Sequence executors over server, pod and pods: ReduceScatter from the top level down (NHR across pods, NHR across
    the servers of a pod, mesh in the server), AllGather from the bottom up."""
    comms = make(n, topo=topo, algo="level0:NA;level1:NHR;level2:NHR")
    for count in (1, 5, 977, 30011):
        ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int32) for r in range(n)]
        ag_out = [np.zeros(count * n, np.int32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
        assert comms[0].last_algorithm() == "HostAllGatherSequenceMeshNHRNHR", comms[0].last_algorithm()
        for o in ag_out:
            assert np.array_equal(o, np.concatenate(ag_in))
        rs_in = [np.random.default_rng(40 + r).standard_normal(count * n) for r in range(n)]
        rs_out = [np.zeros(count, np.float64) for _ in range(n)]
        verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
        assert comms[0].last_algorithm() == "HostReduceScatterSequenceMeshNHRNHR", comms[0].last_algorithm()
        ref = np.sum(np.stack(rs_in), 0)
        for r in range(n):
            np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=1e-12, atol=1e-13)
    destroy(comms)


@pytest.mark.parametrize("n", [4, 6, 7, 8, 12])
def test_all_reduce_on_a_squeezed_grid(algo_env, n):
    """A flat group folded into rows x columns (squeeze 2-D match): mesh ReduceScatter along the rows, mesh AllReduce
    along the columns, mesh AllGather along the rows; a prime count runs as one mesh."""
    comms = make(n, algo="allreduce=level0:hier")
    for count in (1, 77, 10007):
        ins = [np.random.default_rng(200 + r).standard_normal(count).astype(np.float32) for r in range(n)]
        outs = [np.zeros(count, np.float32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        assert comms[0].last_algorithm() == "HostAllReduceSequenceSqueeze2DMeshMesh", comms[0].last_algorithm()
        ref = np.sum(np.stack(ins).astype(np.float64), 0)
        for o in outs:
            np.testing.assert_allclose(o, ref, rtol=3e-6, atol=3e-5)
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
    destroy(comms)


@pytest.mark.parametrize("n", [2, 5, 8])
def test_mesh_with_a_detour(algo_env, n):
    """AllGather, ReduceScatter and Scatter whose pair transfers are split over two channels (queues) by bandwidth:
    p - 1 mesh links against 8 ports of the second link class unless the split-ratio variable says otherwise."""
    comms = make(n, algo="allgather=level0:detour/reducescatter=level0:detour/scatter=level0:detour")
    try:
        for ratio in (None, "1,3", "1,0"):
            if ratio:
                os.environ["HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO"] = ratio
            else:
                os.environ.pop("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", None)
            lib.HcclReloadEnvConfig()
            for count in (1, 130, 4099):
                ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int32) for r in range(n)]
                ag_out = [np.zeros(count * n, np.int32) for _ in range(n)]
                verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
                assert comms[0].last_algorithm() == "HostAllGatherSoleMeshZAxisDetour", comms[0].last_algorithm()
                for o in ag_out:
                    assert np.array_equal(o, np.concatenate(ag_in))
                rs_in = [np.random.default_rng(50 + r).standard_normal(count * n) for r in range(n)]
                rs_out = [np.zeros(count, np.float64) for _ in range(n)]
                verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
                assert comms[0].last_algorithm() == "HostReduceScatterSoleMeshZAxisDetour", comms[0].last_algorithm()
                ref = np.sum(np.stack(rs_in), 0)
                for r in range(n):
                    np.testing.assert_allclose(rs_out[r], ref[r * count:(r + 1) * count], rtol=1e-12, atol=1e-13)
                for root in (0, n - 1):
                    sc_in = [np.arange(count * n, dtype=np.int64) + 1000 * r for r in range(n)]
                    sc_out = [np.zeros(count, np.int64) for _ in range(n)]
                    verified(comms, lambda r, c: c.scatter(sc_in[r], sc_out[r], root))
                    assert comms[0].last_algorithm() == "HostScatterSoleMeshZAxisDetour", comms[0].last_algorithm()
                    for r in range(n):
                        assert np.array_equal(sc_out[r], sc_in[root][r * count:(r + 1) * count])
    finally:
        os.environ.pop("HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO", None)
        lib.HcclReloadEnvConfig()
    destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 6, 8, 11])
def test_nonuniform_bruck(algo_env, n):
    comms = make(n, algo="level0:NA;level1:NB")
    for count in (1, 77, 1025):
        ag_in = [np.random.default_rng(r).integers(-9, 9, count).astype(np.int32) for r in range(n)]
        ag_out = [np.zeros(count * n, np.int32) for _ in range(n)]
        verified(comms, lambda r, c: c.all_gather(ag_in[r], ag_out[r]))
        assert comms[0].last_algorithm().endswith("NB")
        for o in ag_out:
            assert np.array_equal(o, np.concatenate(ag_in))
        for root in (0, n // 2):
            bufs = [np.full(count, r, np.float32) for r in range(n)]
            verified(comms, lambda r, c: c.broadcast(bufs[r], root))
            assert comms[0].last_algorithm().endswith("NB")
            assert all(np.all(b == root) for b in bufs)
            src = np.arange(count * n, dtype=np.int32)
            outs = [np.zeros(count, np.int32) for _ in range(n)]
            verified(comms, lambda r, c: c.scatter(src if r == root else None, outs[r], root))
            assert comms[0].last_algorithm().endswith("NB")
            for r, o in enumerate(outs):
                assert np.array_equal(o, src[r * count:(r + 1) * count])
    destroy(comms)


@pytest.mark.parametrize("topo,n", [(TWO_BY_FOUR, 8), (THREE_BY_TWO, 6), (None, 4)])
def test_hierarchical_alltoall(algo_env, topo, n):
    comms = make(n, topo=topo, algo="level0:NA;level1:hier")
    count = 129
    a2a_in = [np.arange(count * n, dtype=np.int64) + 1000000 * r for r in range(n)]
    a2a_out = [np.zeros(count * n, np.int64) for _ in range(n)]
    verified(comms, lambda r, c: c.all_to_all(a2a_in[r], a2a_out[r]))
    if topo:
        assert "Hier" in comms[0].last_algorithm(), comms[0].last_algorithm()
    for r in range(n):
        for q in range(n):
            assert np.array_equal(a2a_out[r][q * count:(q + 1) * count], a2a_in[q][r * count:(r + 1) * count])
    # variable counts, zero-sized blocks included
    cnt = [[(i * 5 + j * 3) % 7 for j in range(n)] for i in range(n)]
    sends = [np.arange(max(1, sum(cnt[i])), dtype=np.float32) + 1000 * i for i in range(n)]
    recvs = [np.zeros(max(1, sum(cnt[j][i] for j in range(n))), np.float32) for i in range(n)]
    recvs2 = [np.zeros_like(x) for x in recvs]

    def a2av(i, c):
        sd = [sum(cnt[i][:j]) for j in range(n)]
        rc = [cnt[j][i] for j in range(n)]
        rd = [sum(rc[:j]) for j in range(n)]
        c.all_to_all_v(sends[i], cnt[i], sd, recvs[i], rc, rd)

    verified(comms, a2av)
    verified(comms, lambda i, c: c.all_to_all_vc(sends[i], cnt, recvs2[i]))
    if topo:
        assert "Hier" in comms[0].last_algorithm()
    for i in range(n):
        off = 0
        for j in range(n):
            sd = sum(cnt[j][:i])
            assert np.array_equal(recvs[i][off:off + cnt[j][i]], sends[j][sd:sd + cnt[j][i]])
            off += cnt[j][i]
        assert np.array_equal(recvs[i], recvs2[i])
    destroy(comms)


@pytest.mark.parametrize("topo,n", [(TWO_BY_FOUR, 8), (THREE_BY_TWO, 6)])
def test_two_level_rooted_operators(algo_env, topo, n):
    comms = make(n, topo=topo, algo="broadcast=level0:NA;level1:NHR/reduce=level0:NA;level1:NHR/scatter=level0:NA;level1:hier/barrier=level0:NA;level1:hier")
    for count in (1, 50, 3001):
        for root in (0, 1, n - 1):
            bufs = [np.full(count, 7 * r + 1, np.int32) for r in range(n)]
            verified(comms, lambda r, c: c.broadcast(bufs[r], root))
            assert "Sequence" in comms[0].last_algorithm(), comms[0].last_algorithm()
            assert all(np.all(b == 7 * root + 1) for b in bufs)
            ins = [np.random.default_rng(r).standard_normal(count) for r in range(n)]
            out = np.zeros(count)
            verified(comms, lambda r, c: c.reduce(ins[r], out if r == root else None, root))
            assert "Sequence" in comms[0].last_algorithm()
            np.testing.assert_allclose(out, np.sum(np.stack(ins), 0), rtol=1e-12, atol=1e-13)
            src = np.arange(count * n, dtype=np.int16)
            outs = [np.zeros(count, np.int16) for _ in range(n)]
            verified(comms, lambda r, c: c.scatter(src if r == root else None, outs[r], root))
            assert "Sequence" in comms[0].last_algorithm()
            for r, o in enumerate(outs):
                assert np.array_equal(o, src[r * count:(r + 1) * count])
    verified(comms, lambda r, c: c.barrier())
    assert "Sequence" in comms[0].last_algorithm()
    destroy(comms)


TREES = [
    (None, 5, "nhr"),
    (None, 6, "par(mesh,ring)"),
    (None, 7, "par(nb,rhd,3:1)"),
    (TWO_BY_FOUR, 8, "seq(mesh,nhr)"),
    (TWO_BY_FOUR, 8, "par(seq(mesh,nhr),rev(seq(nhr,mesh)))"),
    (TWO_BY_FOUR, 8, "rev(seq(ring,mesh))"),
    (THREE_BY_TWO, 6, "seq(mesh,par(ring,nb,1:1))"),
    (THREE_BY_TWO, 6, "rhd"),
    (TWO_PODS, 8, "seq(mesh,nhr,ring)"),
    (TWO_PODS, 8, "seq(mesh,rhd)"),
    (TWO_PODS, 8, "par(seq(mesh,ring,nhr),rev(seq(nhr,nb,mesh)),2:1)"),
]


@pytest.mark.parametrize("topo,n,tree", TREES)
def test_tree_executor(algo_env, topo, n, tree):
    os.environ["HCCL_ALGO_TREE"] = tree
    try:
        comms = make(n, topo=topo, algo="allreduce=level0:tree")
        for count in (1, 97, 5003):
            ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
            outs = [np.zeros(count, np.float32) for _ in range(n)]
            verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
            assert comms[0].last_algorithm() == "HostAllReduceTree"
            ref = np.sum(np.stack(ins).astype(np.float64), 0)
            for o in outs:
                np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
        destroy(comms)
    finally:
        os.environ.pop("HCCL_ALGO_TREE")
        lib.HcclReloadEnvConfig()


def test_tree_executor_is_not_selected_without_a_tree_and_rejects_too_deep_a_tree(algo_env):
    comms = make(4, algo="allreduce=level0:tree")
    ins = [np.full(10, r, np.float32) for r in range(4)]
    outs = [np.zeros(10, np.float32) for _ in range(4)]
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
    assert "Tree" not in comms[0].last_algorithm() and np.all(outs[0] == 6)
    destroy(comms)
    os.environ["HCCL_ALGO_TREE"] = "seq(mesh,nhr)"
    try:
        comms = make(4, algo="allreduce=level0:tree")      # one-level topology, two-level tree
        with pytest.raises(hb.HcclError):
            run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
        destroy(comms)
    finally:
        os.environ.pop("HCCL_ALGO_TREE")
        lib.HcclReloadEnvConfig()


def test_servers_of_different_sizes_fall_back_to_flat_algorithms(algo_env):
    n = 5
    comms = make(n, topo="[[[0,1,2],[3,4]]]", algo=None)
    count = 777
    ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
    outs = [np.zeros(count, np.float32) for _ in range(n)]
    verified(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
    name = comms[0].last_algorithm()
    assert "Sole" in name or "Concurrent" in name, name
    ref = np.sum(np.stack(ins).astype(np.float64), 0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
    bufs = [np.full(count, r, np.int32) for r in range(n)]
    verified(comms, lambda r, c: c.broadcast(bufs[r], 4))
    assert all(np.all(b == 4) for b in bufs)
    rs_in = [np.random.default_rng(5 + r).standard_normal(16 * n).astype(np.float32) for r in range(n)]
    rs_out = [np.zeros(16, np.float32) for _ in range(n)]
    verified(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
    ref = np.sum(np.stack(rs_in).astype(np.float64), 0)
    for r in range(n):
        np.testing.assert_allclose(rs_out[r], ref[r * 16:(r + 1) * 16], rtol=2e-6, atol=2e-5)
    destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 5, 8])
@pytest.mark.parametrize("key,tag", [("level0:NA;level1:ring", "Ring"), ("level0:NA;level1:NHR", "NHR"), ("level0:NA;level1:H-D_R", "RHD"),
                                     ("level0:NA;level1:fullmesh", "Mesh")])
def test_v_operators_on_every_template(algo_env, n, key, tag):
    """AllGatherV and ReduceScatterV with unequal, gapped and empty blocks through ring, NHR, RHD and mesh."""
    comms = make(n, algo=key)
    counts = [(3 * r + 1) % 5 * 7 for r in range(n)]              # some blocks are empty
    if sum(counts) == 0:
        counts[0] = 4
    displs = [sum(counts[:r]) + 3 * r for r in range(n)]          # gaps between the blocks
    total = displs[-1] + counts[-1]
    ins = [np.full(counts[r], r + 1, np.float32) for r in range(n)]
    outs = [np.full(total, -1, np.float32) for _ in range(n)]
    verified(comms, lambda r, c: c.all_gather_v(ins[r], outs[r], counts, displs))
    assert comms[0].last_algorithm() == f"HostAllGatherVSole{tag}", comms[0].last_algorithm()
    for o in outs:
        for r in range(n):
            assert np.all(o[displs[r]:displs[r] + counts[r]] == r + 1)
        gaps = np.ones(total, bool)
        for r in range(n):
            gaps[displs[r]:displs[r] + counts[r]] = False
        assert np.all(o[gaps] == -1)                              # nothing written between the blocks
    sends = [np.random.default_rng(r).integers(-20, 20, total).astype(np.int64) for r in range(n)]
    recvs = [np.zeros(counts[r], np.int64) for r in range(n)]
    verified(comms, lambda r, c: c.reduce_scatter_v(sends[r], recvs[r], counts, displs))
    assert comms[0].last_algorithm() == f"HostReduceScatterVSole{tag}", comms[0].last_algorithm()
    ref = np.sum(np.stack(sends), 0)
    for r in range(n):
        assert np.array_equal(recvs[r], ref[displs[r]:displs[r] + counts[r]])
    destroy(comms)


@pytest.mark.parametrize("n", [2, 3, 6, 8])
@pytest.mark.parametrize("key,tag", [("level0:NA;level1:ring", "Ring"), ("level0:NA;level1:H-D_R", "RHD")])
def test_rooted_operators_on_ring_and_halving_doubling(algo_env, n, key, tag):
    comms = make(n, algo=key)
    for count in (1, 77, 2050):
        for root in (0, n - 1):
            bufs = [np.full(count, 3 * r + 1, np.int32) for r in range(n)]
            verified(comms, lambda r, c: c.broadcast(bufs[r], root))
            assert comms[0].last_algorithm() == f"HostBroadcastSole{tag}", comms[0].last_algorithm()
            assert all(np.all(b == 3 * root + 1) for b in bufs)
            ins = [np.random.default_rng(r).standard_normal(count) for r in range(n)]
            out = np.zeros(count)
            verified(comms, lambda r, c: c.reduce(ins[r], out if r == root else None, root))
            assert comms[0].last_algorithm() == f"HostReduceSole{tag}", comms[0].last_algorithm()
            np.testing.assert_allclose(out, np.sum(np.stack(ins), 0), rtol=1e-12, atol=1e-13)
    destroy(comms)
