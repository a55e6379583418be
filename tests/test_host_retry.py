"""Operator retry on the host engine: a dropped notify makes an attempt time
out on every rank; with HCCL_OP_RETRY_ENABLE the ranks meet at the recovery
point and issue the operator again from its input.  All failures are made on
the host (a message the test drops, a rank that stays away)."""
import ctypes
import os
import threading

import numpy as np
import pytest

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200._lib import lib

from test_host_engine import run_ranks


@pytest.fixture
def retry_env():
    keys = ("HCCL_OP_RETRY_ENABLE", "HCCL_OP_RETRY_PARAMS", "HCCL_ALGO")
    old = {k: os.environ.get(k) for k in keys}
    yield
    for k, v in old.items():
        if v is None:
            os.environ.pop(k, None)
        else:
            os.environ[k] = v
    lib.HcclReloadEnvConfig()


def make(n, enable, params=None, timeout_ms=800):
    os.environ.pop("HCCL_ALGO", None)
    os.environ["HCCL_OP_RETRY_ENABLE"] = enable
    if params:
        os.environ["HCCL_OP_RETRY_PARAMS"] = params
    else:
        os.environ.pop("HCCL_OP_RETRY_PARAMS", None)
    lib.HcclReloadEnvConfig()
    return Communicator.host_sim(n, None, hb.make_config(buffer_mib=8, exec_timeout_ms=timeout_ms))


def recoveries(comm):
    v = ctypes.c_uint64(0)
    assert lib.HcclTestHostRecoveries(comm._h, ctypes.byref(v)) == 0
    return v.value


def test_dropped_notify_is_retried_and_the_result_is_right(retry_env):
    n, count = 4, 3001
    comms = make(n, "L1:1", "MaxCnt:2,HoldTime:5,IntervalTime:5")
    ins = [np.random.default_rng(r).standard_normal(count).astype(np.float32) for r in range(n)]
    outs = [np.zeros(count, np.float32) for _ in range(n)]
    assert lib.HcclTestHostDropPosts(comms[2]._h, 1) == 0
    run_ranks(comms, lambda r, c: c.all_reduce(ins[r], outs[r]))
    assert recoveries(comms[0]) == 1
    ref = np.sum(np.stack(ins).astype(np.float64), 0)
    for o in outs:
        np.testing.assert_allclose(o, ref, rtol=2e-6, atol=2e-5)
    # the communicator stays usable, and a clean call does not go through the recovery point
    rs_in = [np.full(8 * n, r + 1.0) for r in range(n)]
    rs_out = [np.zeros(8) for _ in range(n)]
    run_ranks(comms, lambda r, c: c.reduce_scatter(rs_in[r], rs_out[r]))
    assert all(np.all(o == 10) for o in rs_out) and recoveries(comms[0]) == 1
    for c in comms:
        c.destroy()


def test_retry_gives_up_after_max_count(retry_env):
    n = 3
    comms = make(n, "L1:1", "MaxCnt:1,HoldTime:0,IntervalTime:0", timeout_ms=600)
    ins = [np.ones(64, np.float32) for _ in range(n)]
    outs = [np.zeros(64, np.float32) for _ in range(n)]
    assert lib.HcclTestHostDropPosts(comms[0]._h, 1000) == 0      # every attempt loses its messages
    codes = [None] * n

    def body(r, c):
        try:
            c.all_reduce(ins[r], outs[r])
        except hb.HcclError as e:
            codes[r] = e.code

    run_ranks(comms, body)
    assert all(code == hb.Result.E_OPRETRY_FAIL for code in codes), codes
    assert recoveries(comms[0]) == 1
    for c in comms:
        c.destroy()


def test_without_retry_or_in_place_the_failure_is_reported(retry_env):
    n = 3
    for enable, in_place in (("L1:0", False), ("L1:1", True)):
        comms = make(n, enable, timeout_ms=600)
        ins = [np.ones(64, np.float32) for _ in range(n)]
        outs = [np.zeros(64, np.float32) for _ in range(n)]
        assert lib.HcclTestHostDropPosts(comms[1]._h, 1) == 0
        codes = [None] * n

        def body(r, c):
            try:
                c.all_reduce(ins[r], ins[r] if in_place else outs[r])
            except hb.HcclError as e:
                codes[r] = e.code

        run_ranks(comms, body)
        assert all(code in (hb.Result.E_TIMEOUT, hb.Result.E_REMOTE) for code in codes), codes
        assert recoveries(comms[0]) == 0
        for c in comms:
            c.destroy()
