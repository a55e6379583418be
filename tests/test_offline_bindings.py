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


def test_sweep_rows_render_as_markdown_and_feed_the_link_model(tmp_path):
    """The offline halves of the measurement tools: `bench/sweep.py --from-jsonl` renders saved rows (every fourth size
    with --ladder), `bench/link_model.py` turns symmetric AllGather / switch AllReduce rows into utilisation curves per
    GPU count."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    rows = []
    for i, nbytes in enumerate(1 << s for s in range(20, 29)):
        for impl, alg, t in (("hccl_sym", "P2pAllGatherSoleMesh", 10 + nbytes / 600e3), ("hccl", "P2pAllGatherSoleMesh", 12 + nbytes / 550e3), ("nccl", "nccl", 15 + nbytes / 500e3)):
            rows.append({"op": "all_gather", "dtype": "bf16", "bytes": nbytes, "impl": impl, "time_us": t, "max_us": t * 1.2, "algbw_gbs": nbytes / t / 1e3,
                         "busbw_gbs": nbytes / t / 1e3 * 7 / 8, "n_gpus": 8, "alg": alg})
        rows.append({"op": "all_reduce", "dtype": "bf16", "bytes": nbytes, "impl": "hccl_sym", "time_us": 12 + nbytes / 400e3, "max_us": 20 + nbytes / 400e3,
                     "algbw_gbs": 1.0, "busbw_gbs": 1.0, "n_gpus": 8, "alg": "NvlsAllReduceSoleMesh"})
    src = tmp_path / "rows.jsonl"
    src.write_text("\n".join(json.dumps(r) for r in rows) + "\n")
    md = tmp_path / "sweep.md"
    subprocess.run([sys.executable, str(root / "bench" / "sweep.py"), "--from-jsonl", str(src), "--ladder", "--markdown", str(md), "--command", "the command"],
                   check=True, timeout=120)
    text = md.read_text()
    assert "# Collective sweep against NCCL, 8 x B200" in text and "the command" in text
    table = [line for line in text.splitlines() if line.startswith("| ") and "MiB" in line]
    assert len(table) == 3 and table[0].startswith("| 1 MiB |") and table[-1].startswith("| 256 MiB |")      # sizes 0, 4 and the last of 9
    out = tmp_path / "link_model.json"
    subprocess.run([sys.executable, str(root / "bench" / "link_model.py"), str(src), "--out", str(out)], check=True, timeout=120)
    model = json.loads(out.read_text())
    assert set(model["utilisation"]) == {"p2p", "nvls"} and "8" in model["utilisation"]["p2p"] and "8" in model["utilisation"]["nvls"]
    curve = model["utilisation"]["p2p"]["8"]
    assert all(0 < u <= 1.2 for _, u in curve) and curve[-1][1] > curve[0][1]          # larger messages use the link better
