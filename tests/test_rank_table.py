"""Rank-table (cluster information) loader behind HcclCommInitClusterInfo: HCCL's JSON layout, given as text or as
a file; malformed tables are rejected with the reason in the log."""
import ctypes
import json

from hccl_b200._lib import lib


def render(arg: str) -> str:
    buf = ctypes.create_string_buffer(1 << 14)
    assert lib.HcclDebugStepTable(b"rank_table", 0, 0, arg.encode(), buf, len(buf)) == 0
    return buf.value.decode()


def table(servers=2, per=4, **over):
    t = {"status": "completed", "version": "1.0", "server_count": str(servers), "server_list": []}
    rank = 0
    for s in range(servers):
        devs = []
        for d in range(per):
            devs.append({"device_id": str(d), "device_ip": f"192.168.{s}.{10 + d}", "device_port": str(16666 + d), "rank_id": str(rank)})
            rank += 1
        t["server_list"].append({"server_id": f"10.0.0.{s + 1}", "host_ip": f"10.0.0.{s + 1}", "device": devs})
    t.update(over)
    return t


def test_text_and_file_give_the_same_table(tmp_path):
    t = table()
    text = render(json.dumps(t))
    lines = text.splitlines()
    assert lines[0].startswith("ranks 8 servers 4 4 root 10.0.0.1:16666 fingerprint "), lines[0]
    assert lines[1] == "rank 0 server 10.0.0.1 device 0 ip 192.168.0.10"
    assert lines[8] == "rank 7 server 10.0.0.2 device 3 ip 192.168.1.13"
    path = tmp_path / "ranktable.json"
    path.write_text(json.dumps(t, indent=2))
    assert render(str(path)) == text
    # every rank derives the same communicator id from the same table; another table gives another id
    other = render(json.dumps(table(servers=2, per=2)))
    assert other.splitlines()[0].split()[-1] != lines[0].split()[-1]


def test_explicit_root_and_rank_order():
    t = table(root_ip="127.0.0.1", root_port="61000")
    # devices listed out of rank order are sorted by rank id
    t["server_list"][0]["device"].reverse()
    lines = render(json.dumps(t)).splitlines()
    assert " root 127.0.0.1:61000 " in lines[0]
    assert lines[1].startswith("rank 0 server 10.0.0.1 device 0")


def test_malformed_tables_are_rejected(tmp_path):
    assert render("{not json").startswith("error:")
    assert render(json.dumps(table(status="initializing"))).startswith("error:")
    assert render(json.dumps(table(server_count="3"))).startswith("error:")
    t = table()
    t["server_list"][1]["device"][0]["rank_id"] = "0"                 # duplicate rank id
    assert render(json.dumps(t)).startswith("error:")
    t = table()
    del t["server_list"][0]["device"][2]["device_id"]
    assert render(json.dumps(t)).startswith("error:")
    t = table()
    t["server_list"] = []
    assert render(json.dumps(t)).startswith("error:")
    assert render(str(tmp_path / "missing.json")).startswith("error:")
