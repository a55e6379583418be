"""Offline binding checks (no device): every function the public headers declare is exported by the built library,
the enumerations of the Python layer agree with the C headers, and the structures the binding mirrors have the
sizes the library was compiled with."""
import ctypes
import re
from pathlib import Path

from hccl_b200 import _lib
from hccl_b200._lib import lib
from hccl_b200.types import Cmd, DataType, ReduceOp, Result

INC = Path(__file__).resolve().parent.parent / "csrc" / "include" / "hccl"
DECL = re.compile(r"^\s*(?:HcclResult|uint32_t|uint64_t|const char\*|double|void|int)\s+(Hccl[A-Za-z0-9]+)\s*\(", re.M)


def declared_functions():
    names = set()
    for h in sorted(INC.glob("*.h")):
        if h.name in ("hccl_tuner_plugin.h", "hccl_algo_plugin.h"):
            continue        # implemented by plugins, not by the library
        names |= set(DECL.findall(h.read_text()))
    return names


def test_every_declared_function_is_exported():
    names = declared_functions()
    assert len(names) > 80, len(names)
    missing = sorted(n for n in names if not hasattr(lib, n))
    assert not missing, missing


def enum_values(header: str, prefix: str):
    text = (INC / header).read_text()
    out = {}
    for name, value in re.findall(rf"\b({prefix}[A-Z0-9_]+)\s*=\s*(-?\d+)", text):
        out[name] = int(value)
    return out


def test_python_enums_match_the_headers():
    c_types = enum_values("hccl_types.h", "HCCL_DATA_TYPE_")
    for member in DataType:
        assert c_types[f"HCCL_DATA_TYPE_{member.name}"] == member.value, member
    c_cmds = enum_values("hccl_types.h", "HCCL_CMD_")
    for member in Cmd:
        assert c_cmds[f"HCCL_CMD_{member.name}"] == member.value, member
    c_res = enum_values("hccl_types.h", "HCCL_E_")
    for member in Result:
        if member.name.startswith("E_"):
            assert c_res[f"HCCL_{member.name}"] == member.value, member
    c_ops = enum_values("hccl_types.h", "HCCL_REDUCE_")
    for member in ReduceOp:
        assert c_ops[f"HCCL_REDUCE_{member.name}"] == member.value, member


def test_mirrored_structures_have_the_library_sizes():
    assert ctypes.sizeof(_lib.HcclRootInfo) == _lib.HCCL_ROOT_INFO_BYTES
    assert ctypes.sizeof(_lib.HcclCommConfig) == 2304
    assert ctypes.sizeof(_lib.HcclSendRecvItem) == 32
    assert ctypes.sizeof(_lib.HcclResPackGraphMode) == 40
    text = (INC / "hccl_comm.h").read_text() + (INC / "hccl_types.h").read_text()
    assert "4108" in text or "HCCL_ROOT_INFO_BYTES" in text
