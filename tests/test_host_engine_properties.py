"""Property tests of the host engine: for any rank count, message size, algorithm preference, data type and root, an
operator gives the NumPy result and its recorded trace passes the verifier."""
import numpy as np
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from hccl_b200 import ReduceOp

import os

import pytest

from hccl_b200._lib import lib

from test_host_engine import destroy, make, run_ranks


@pytest.fixture(autouse=True)
def restore_algo_preference():
    old = os.environ.get("HCCL_ALGO")
    yield
    if old is None:
        os.environ.pop("HCCL_ALGO", None)
    else:
        os.environ["HCCL_ALGO"] = old
    lib.HcclReloadEnvConfig()


PREFS = [None, "level0:NA;level1:ring", "level0:NA;level1:NHR", "level0:NA;level1:H-D_R", "level0:NA;level1:fullmesh", "level0:NA;level1:NB",
         "level0:NA;level1:concurrent", "level0:NA;level1:oneshot", "level0:NA;level1:serial", "level0:NA;level1:2die",
         "level0:NA;level1:meshconcur", "level0:NA;level1:detour"]
DTYPES = [np.int32, np.int64, np.float64]
FOLD = {ReduceOp.SUM: np.add, ReduceOp.MAX: np.maximum, ReduceOp.MIN: np.minimum}


@settings(max_examples=80, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(n=st.integers(2, 7), count=st.integers(1, 1500), pref=st.sampled_from(PREFS), dtype=st.sampled_from(DTYPES),
       op=st.sampled_from(list(FOLD)), seed=st.integers(0, 1000))
def test_allreduce_any_shape(n, count, pref, dtype, op, seed):
    rng = np.random.default_rng(seed)
    ins = [rng.integers(-50, 50, count).astype(dtype) for _ in range(n)]
    outs = [np.zeros(count, dtype) for _ in range(n)]
    comms = make(n, algo=pref, buffer_mib=2)
    comms[0].trace_begin()
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r], op))
    rep = comms[0].trace_verify()
    destroy(comms)
    assert rep.startswith("OK"), rep
    want = ins[0].copy()
    for x in ins[1:]:
        want = FOLD[op](want, x)
    for o in outs:
        assert np.array_equal(o, want)


@settings(max_examples=80, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(n=st.integers(2, 7), count=st.integers(1, 700), pref=st.sampled_from(PREFS), kind=st.sampled_from(["ag", "rs", "bc", "sc", "a2a", "red"]),
       root=st.integers(0, 6), seed=st.integers(0, 1000))
def test_other_operators_any_shape(n, count, pref, kind, root, seed):
    root %= n
    rng = np.random.default_rng(seed)
    comms = make(n, algo=pref, buffer_mib=2)
    wide = [rng.integers(-50, 50, count * n).astype(np.int64) for _ in range(n)]
    narrow = [w[:count].copy() for w in wide]
    outs = {}

    def body(r, c):
        if kind == "ag":
            outs[r] = np.zeros(count * n, np.int64)
            c.all_gather(narrow[r], outs[r])
        elif kind == "rs":
            outs[r] = np.zeros(count, np.int64)
            c.reduce_scatter(wide[r], outs[r])
        elif kind == "bc":
            outs[r] = narrow[r].copy()
            c.broadcast(outs[r], root)
        elif kind == "sc":
            outs[r] = np.zeros(count, np.int64)
            c.scatter(wide[root] if r == root else None, outs[r], root)
        elif kind == "a2a":
            outs[r] = np.zeros(count * n, np.int64)
            c.all_to_all(wide[r], outs[r])
        else:
            outs[r] = np.zeros(count, np.int64)
            c.reduce(narrow[r], outs[r] if r == root else None, root)

    comms[0].trace_begin()
    run_ranks(comms, body)
    rep = comms[0].trace_verify()
    destroy(comms)
    assert rep.startswith("OK"), rep
    total = np.sum(np.stack(wide), 0)
    for r in range(n):
        if kind == "ag":
            assert np.array_equal(outs[r], np.concatenate(narrow))
        elif kind == "rs":
            assert np.array_equal(outs[r], total[r * count:(r + 1) * count])
        elif kind == "bc":
            assert np.array_equal(outs[r], narrow[root])
        elif kind == "sc":
            assert np.array_equal(outs[r], wide[root][r * count:(r + 1) * count])
        elif kind == "a2a":
            assert np.array_equal(outs[r], np.concatenate([wide[q][r * count:(r + 1) * count] for q in range(n)]))
        elif r == root:
            assert np.array_equal(outs[r], np.sum(np.stack(narrow), 0))


def _topology(shape):
    """Topology literal and rank count for (servers per pod..., ranks per server): (2, 4) -> two servers of four,
    (2, 2, 3) -> two pods of two servers of three."""
    if len(shape) == 2:
        servers, per = shape
        rows = [list(range(s * per, (s + 1) * per)) for s in range(servers)]
        return "[" + str(rows).replace(" ", "") + "]", servers * per
    pods, servers, per = shape
    lit, r = [], 0
    for _ in range(pods):
        pod = []
        for _ in range(servers):
            pod.append(list(range(r, r + per)))
            r += per
        lit.append(pod)
    return str(lit).replace(" ", ""), r


HIER_PREFS = [None, "level0:NA;level1:NHR", "level0:NA;level1:ring", "level0:NA;level1:H-D_R", "level0:NA;level1:pipeline", "level0:NA;level1:omnipipe",
              "level0:NA;level1:NHR;level2:NHR", "level0:NA;level1:omnipipe;level2:omnipipe", "level0:NA;level1:hier"]
SHAPES = [(2, 2), (2, 3), (3, 2), (2, 4), (3, 3), (4, 2), (2, 2, 2), (2, 2, 3), (3, 2, 2)]


@settings(max_examples=120, deadline=None, suppress_health_check=[HealthCheck.too_slow])
@given(shape=st.sampled_from(SHAPES), count=st.integers(1, 900), pref=st.sampled_from(HIER_PREFS),
       kind=st.sampled_from(["ar", "ag", "rs", "bc", "sc", "a2a", "red"]), root=st.integers(0, 17), seed=st.integers(0, 1000))
def test_operators_on_hierarchical_topologies(shape, count, pref, kind, root, seed):
    """Servers and pods of any of these shapes, every executor family the preference can name (Sequence on two and
    three levels, Parallel, Pipeline on two and three levels, hierarchical AlltoAll), every operator and root: the
    NumPy result, and a trace the verifier accepts."""
    topo, n = _topology(shape)
    root %= n
    rng = np.random.default_rng(seed)
    comms = make(n, topo=topo, algo=pref, buffer_mib=2)
    wide = [rng.integers(-50, 50, count * n).astype(np.int64) for _ in range(n)]
    narrow = [w[:count].copy() for w in wide]
    outs = {}

    def body(r, c):
        if kind == "ar":
            outs[r] = np.zeros(count, np.int64)
            c.all_reduce(narrow[r], outs[r])
        elif kind == "ag":
            outs[r] = np.zeros(count * n, np.int64)
            c.all_gather(narrow[r], outs[r])
        elif kind == "rs":
            outs[r] = np.zeros(count, np.int64)
            c.reduce_scatter(wide[r], outs[r])
        elif kind == "bc":
            outs[r] = narrow[r].copy()
            c.broadcast(outs[r], root)
        elif kind == "sc":
            outs[r] = np.zeros(count, np.int64)
            c.scatter(wide[root] if r == root else None, outs[r], root)
        elif kind == "a2a":
            outs[r] = np.zeros(count * n, np.int64)
            c.all_to_all(wide[r], outs[r])
        else:
            outs[r] = np.zeros(count, np.int64)
            c.reduce(narrow[r], outs[r] if r == root else None, root)

    comms[0].trace_begin()
    run_ranks(comms, body)
    rep = comms[0].trace_verify()
    name = comms[0].last_algorithm()
    destroy(comms)
    assert rep.startswith("OK"), (name, rep)
    total = np.sum(np.stack(wide), 0)
    for r in range(n):
        if kind == "ar":
            assert np.array_equal(outs[r], np.sum(np.stack(narrow), 0)), name
        elif kind == "ag":
            assert np.array_equal(outs[r], np.concatenate(narrow)), name
        elif kind == "rs":
            assert np.array_equal(outs[r], total[r * count:(r + 1) * count]), name
        elif kind == "bc":
            assert np.array_equal(outs[r], narrow[root]), name
        elif kind == "sc":
            assert np.array_equal(outs[r], wide[root][r * count:(r + 1) * count]), name
        elif kind == "a2a":
            assert np.array_equal(outs[r], np.concatenate([wide[q][r * count:(r + 1) * count] for q in range(n)])), name
        elif r == root:
            assert np.array_equal(outs[r], np.sum(np.stack(narrow), 0)), name
