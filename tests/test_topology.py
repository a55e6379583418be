"""Topology model and match: what a three-level literal gives each rank, the groups of the one / two / three level
matches, servers of different sizes, and the guards of the serialised form."""
import ctypes

import pytest

from hccl_b200._lib import lib


def topo(js, n, rank, kind):
    lib.HcclDebugTopo.restype = ctypes.c_int
    lib.HcclDebugTopo.argtypes = [ctypes.c_char_p, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_char_p, ctypes.c_uint32]
    buf = ctypes.create_string_buffer(1 << 14)
    rc = lib.HcclDebugTopo(js.encode() if js else None, n, rank, kind, buf, len(buf))
    assert rc == 0, rc
    return buf.value.decode().splitlines()


def test_one_server_is_one_flat_group():
    lines = topo(None, 4, 2, 0)
    assert lines[0].startswith("4 ranks, 1 server(s) x 4, 1 pod(s), level0 MESH_1D")
    assert lines[1] == "server 0 pod 0 local 2 symmetric 1 level1Nhr 0"
    assert lines[2] == "level 0: [0,1,2,3]"
    assert lines[-1] == "roundtrip 1 damaged 0 truncated 0"


@pytest.mark.parametrize("rank", range(8))
def test_two_level_match_groups_by_server_and_by_local_index(rank):
    lines = topo("[[[0,1,2,3],[4,5,6,7]]]", 8, rank, 1)
    assert lines[1] == f"server {rank // 4} pod 0 local {rank % 4} symmetric 1 level1Nhr 0"
    assert lines[2] == "level 0: [0,1,2,3] [4,5,6,7]"
    assert lines[3] == "level 1: [0,4] [1,5] [2,6] [3,7]"
    # a one-level match of the same topology ignores the servers
    assert topo("[[[0,1,2,3],[4,5,6,7]]]", 8, rank, 0)[2] == "level 0: [0,1,2,3,4,5,6,7]"


def test_three_level_match_adds_the_pod_level():
    lines = topo("[[[0,1],[2,3]],[[4,5],[6,7]]]", 8, 6, 2)
    assert "4 server(s) x 2, 2 pod(s)" in lines[0]
    assert lines[1] == "server 3 pod 1 local 0 symmetric 1 level1Nhr 0"
    assert lines[2:5] == ["level 0: [0,1] [2,3] [4,5] [6,7]", "level 1: [0,2] [1,3] [4,6] [5,7]", "level 2: [0,4] [1,5] [2,6] [3,7]"]


def test_servers_of_different_sizes_have_no_multi_level_match():
    lines = topo("[[[0,1,2],[3,4]]]", 5, 4, 1)
    assert "(asymmetric)" in lines[0]
    assert lines[1] == "server 1 pod 0 local 1 symmetric 0 level1Nhr 1"        # sizes 3 and 2 share no divisor
    assert lines[2] == "match: HCCL_E_NOT_SUPPORT"
    assert topo("[[[0,1,2],[3,4]]]", 5, 4, 0)[2] == "level 0: [0,1,2,3,4]"      # the flat match still works
    assert topo("[[[0,1,2,3],[4,5]]]", 6, 0, 0)[1].endswith("symmetric 0 level1Nhr 0")   # 4 and 2 share the divisor 2


def test_bad_literals_are_reported():
    assert topo("[[[0,1],[2]]", 3, 0, 0)[0].startswith("error:")
    assert topo("[[0,1,2]]", 3, 0, 0)[0].startswith("error:")
    assert topo("[[[0,1],[2,3]]]", 5, 0, 0)[0].startswith("error:")              # four devices listed, five ranks asked for


def test_squeeze_2d_folds_one_level_into_a_grid():
    """One physical level laid out as rows x columns: the largest divisor that is at most the square root gives the
    number of rows; a prime count stays one group; more than one server is refused."""
    assert topo(None, 8, 3, 3)[2:4] == ["level 0: [0,1,2,3] [4,5,6,7]", "level 1: [0,4] [1,5] [2,6] [3,7]"]
    assert topo(None, 6, 0, 3)[2:4] == ["level 0: [0,1,2] [3,4,5]", "level 1: [0,3] [1,4] [2,5]"]
    assert topo(None, 16, 0, 3)[2:4] == ["level 0: [0,1,2,3] [4,5,6,7] [8,9,10,11] [12,13,14,15]", "level 1: [0,4,8,12] [1,5,9,13] [2,6,10,14] [3,7,11,15]"]
    assert topo(None, 7, 0, 3)[2] == "level 0: [0,1,2,3,4,5,6]"
    assert topo("[[[0,1],[2,3]]]", 4, 0, 3)[2] == "match: HCCL_E_NOT_SUPPORT"
