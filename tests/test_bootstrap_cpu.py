"""The out-of-band bootstrap without a device: rendezvous, all-gather, barrier and agreement between ranks that run as
threads, and the failure paths made on the host - a rank that never joins, a rank that leaves, an injected connection
drop."""
import ctypes
import threading
import time

import pytest

from hccl_b200 import _lib
from hccl_b200._lib import lib
from hccl_b200.types import Result

for name, args in (("HcclDebugBootstrapConnect", [ctypes.POINTER(_lib.HcclRootInfo), ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.POINTER(ctypes.c_void_p)]),
                   ("HcclDebugBootstrapAllGather", [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_uint64]),
                   ("HcclDebugBootstrapBarrier", [ctypes.c_void_p]),
                   ("HcclDebugBootstrapAgree", [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int)]),
                   ("HcclDebugBootstrapInjectFailure", [ctypes.c_void_p]),
                   ("HcclDebugBootstrapClose", [ctypes.c_void_p])):
    if hasattr(lib, name):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = args


def root_info():
    info = _lib.HcclRootInfo()
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == 0
    return info


def run(n, fn):
    out, errs = [None] * n, []

    def body(r):
        try:
            out[r] = fn(r)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)

    ts = [threading.Thread(target=body, args=(r,)) for r in range(n)]
    [t.start() for t in ts]
    [t.join() for t in ts]
    if errs:
        raise errs[0]
    return out


def connect(info, rank, n, timeout_s=20):
    h = ctypes.c_void_p()
    rc = lib.HcclDebugBootstrapConnect(ctypes.byref(info), rank, n, timeout_s, ctypes.byref(h))
    return rc, h


def test_rendezvous_allgather_barrier_and_agreement():
    n = 5
    info = root_info()

    def body(r):
        rc, h = connect(info, r, n)
        assert rc == 0, Result(rc)
        send = (ctypes.c_uint64 * 2)(r, r * r)
        recv = (ctypes.c_uint64 * (2 * n))()
        assert lib.HcclDebugBootstrapAllGather(h, send, recv, 16) == 0
        assert list(recv) == [x for q in range(n) for x in (q, q * q)]
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        all_ok = ctypes.c_int(-1)
        assert lib.HcclDebugBootstrapAgree(h, 1, ctypes.byref(all_ok)) == 0 and all_ok.value == 1
        # one rank says no: everybody learns it (the fallback agreement)
        assert lib.HcclDebugBootstrapAgree(h, 0 if r == 3 else 1, ctypes.byref(all_ok)) == 0 and all_ok.value == 0
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        assert lib.HcclDebugBootstrapClose(h) == 0
        return True

    assert all(run(n, body))


def test_a_rank_that_never_joins_times_the_others_out():
    n = 3
    info = root_info()
    t0 = time.time()

    def body(r):
        if r == 2:
            return "stayed away"
        rc, h = connect(info, r, n, timeout_s=2)
        if rc == 0:                                  # connected to the relay; the rendezvous itself must then fail
            rc = lib.HcclDebugBootstrapBarrier(h)
            lib.HcclDebugBootstrapClose(h)
        return rc

    out = run(n, body)
    assert out[0] == Result.E_TIMEOUT and out[1] == Result.E_TIMEOUT, out
    assert time.time() - t0 < 30


def test_a_rank_that_leaves_is_noticed_by_the_others():
    n = 3
    info = root_info()
    gate = threading.Barrier(n)

    def body(r):
        rc, h = connect(info, r, n)
        assert rc == 0
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        gate.wait()
        if r == 1:
            lib.HcclDebugBootstrapClose(h)           # leaves between two steps
            return "left"
        time.sleep(0.3)
        rc = lib.HcclDebugBootstrapBarrier(h)
        lib.HcclDebugBootstrapClose(h)
        return rc

    out = run(n, body)
    assert out[1] == "left" and out[0] == Result.E_REMOTE and out[2] == Result.E_REMOTE, out


def test_injected_connection_drop_fails_the_next_exchange_only_on_that_rank_first():
    n = 2
    info = root_info()

    def body(r):
        rc, h = connect(info, r, n)
        assert rc == 0
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        if r == 0:
            lib.HcclDebugBootstrapInjectFailure(h)
        send = (ctypes.c_uint32 * 1)(r)
        recv = (ctypes.c_uint32 * n)()
        rc = lib.HcclDebugBootstrapAllGather(h, send, recv, 4)
        lib.HcclDebugBootstrapClose(h)
        return rc

    out = run(n, body)
    assert out[0] != 0, out                           # the rank whose connection dropped
    assert out[1] != 0, out                           # its peer cannot complete the exchange either


def _root_payload(info):
    """(ip, port) of a root info: magic, version, char ip[64], uint32 port, uint64 id."""
    raw = ctypes.string_at(ctypes.addressof(info), 96)
    ip = raw[8:72].split(b"\0")[0].decode()
    port = int.from_bytes(raw[72:76], "little")
    return ip, port


@pytest.fixture
def clean_env():
    import os

    names = ("HCCL_HOST_SOCKET_PORT_RANGE", "HCCL_IF_BASE_PORT", "HCCL_SOCKET_IFNAME", "HCCL_SOCKET_FAMILY", "HCCL_WHITELIST_DISABLE", "HCCL_WHITELIST_FILE", "HCCL_IF_IP")
    old = {k: os.environ.pop(k, None) for k in names}
    lib.HcclReloadEnvConfig()
    yield os.environ
    for k in names:
        os.environ.pop(k, None)
        if old[k] is not None:
            os.environ[k] = old[k]
    lib.HcclReloadEnvConfig()


def test_port_range_interface_rule_and_address_family(clean_env):
    """HCCL_HOST_SOCKET_PORT_RANGE decides the root's port (the first free one of the ranges, before HCCL_IF_BASE_PORT);
    HCCL_SOCKET_IFNAME decides its address; the IPv6 family is refused with a message, not ignored."""
    import socket

    def free(port):
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", port))
                return True
            except OSError:
                return False

    import random

    base = next(b for b in (random.randrange(40000, 60000, 16) for _ in range(200)) if all(free(b + i) for i in range(12)))
    clean_env["HCCL_HOST_SOCKET_PORT_RANGE"] = f"{base}-{base + 3},{base + 8}"
    clean_env["HCCL_IF_BASE_PORT"] = str(base + 11)
    lib.HcclReloadEnvConfig()
    first = root_info()
    assert _root_payload(first) == ("127.0.0.1", base)
    second = root_info()                                  # the first port is taken by the relay of `first`
    assert _root_payload(second)[1] == base + 1
    blocker = socket.socket()
    blocker.bind(("127.0.0.1", base + 2))
    blocker.listen(1)
    assert _root_payload(root_info())[1] == base + 3      # an occupied port is skipped
    assert _root_payload(root_info())[1] == base + 8
    info = _lib.HcclRootInfo()
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == Result.E_TCP_CONNECT      # every listed port is in use
    blocker.close()
    # ranks still meet over a root made this way
    n = 3

    def body(r):
        rc, h = connect(first, r, n)
        assert rc == 0, Result(rc)
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        lib.HcclDebugBootstrapClose(h)

    run(n, body)
    del clean_env["HCCL_HOST_SOCKET_PORT_RANGE"]
    clean_env["HCCL_SOCKET_IFNAME"] = "=lo"
    lib.HcclReloadEnvConfig()
    ip, port = _root_payload(root_info())
    assert ip == "127.0.0.1" and port == base + 11
    clean_env["HCCL_SOCKET_IFNAME"] = "=no_such_nic0"
    lib.HcclReloadEnvConfig()
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == Result.E_NOT_FOUND
    del clean_env["HCCL_SOCKET_IFNAME"], clean_env["HCCL_IF_BASE_PORT"]
    clean_env["HCCL_SOCKET_FAMILY"] = "AF_INET6"
    lib.HcclReloadEnvConfig()
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == Result.E_NOT_SUPPORT


def test_trust_list_admits_only_listed_addresses(clean_env, tmp_path):
    """HCCL_WHITELIST_DISABLE=0: the relay drops connections from addresses that HCCL_WHITELIST_FILE does not list (the
    ranks then time out in Connect); a list with the address lets them in; a missing or malformed file fails the root."""
    n = 2
    wl = tmp_path / "whitelist.json"
    clean_env["HCCL_WHITELIST_DISABLE"] = "0"
    clean_env["HCCL_WHITELIST_FILE"] = str(wl)
    lib.HcclReloadEnvConfig()
    info = _lib.HcclRootInfo()
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == Result.E_PARA                 # no file
    wl.write_text('{"host_ip": ["10.1.2.3", "not-an-address"]}')
    assert lib.HcclGetRootInfo(ctypes.byref(info)) == Result.E_PARA
    wl.write_text('{"host_ip": ["10.1.2.3"], "device_ip": []}')
    closed = root_info()

    def refused(r):
        rc, _ = connect(closed, r, n, timeout_s=2)
        assert rc != 0
    run(n, refused)
    wl.write_text('{"host_ip": ["10.1.2.3", "127.0.0.1"]}')
    opened = root_info()

    def admitted(r):
        rc, h = connect(opened, r, n)
        assert rc == 0, Result(rc)
        assert lib.HcclDebugBootstrapBarrier(h) == 0
        lib.HcclDebugBootstrapClose(h)
    run(n, admitted)
