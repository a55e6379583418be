"""The tuning workflow end to end on the host engine: measure every algorithm
(perf_test.py), keep the fastest per size range (optimize_config.py), and let
the config tuner plugin steer the selector with the result."""
import json
import os
import subprocess
import sys
from pathlib import Path

import hccl_b200 as hb
from hccl_b200._lib import lib
from hccl_b200.types import Cmd, DataType

ROOT = Path(__file__).resolve().parent.parent
EX = ROOT / "examples" / "tuner_plugin"


def test_measure_optimise_and_apply(tmp_path):
    perf = tmp_path / "perf.jsonl"
    env = {k: v for k, v in os.environ.items() if not k.startswith("HCCL_")}
    subprocess.check_call([sys.executable, str(EX / "perf_test.py"), "--host-sim", "4", "--ops", "all_reduce,all_gather", "--sizes", "4096,262144",
                           "--iters", "2", "--out", str(perf)], env=env, stdout=subprocess.DEVNULL)
    rows = [json.loads(l) for l in perf.read_text().splitlines()]
    algs = {r["alg"] for r in rows if r["op"] == "all_reduce"}
    assert {"HostAllReduceSoleRing", "HostAllReduceSoleNHR", "HostAllReduceSoleMeshTwoShot"} <= algs, algs
    tuned = tmp_path / "tuned.json"
    subprocess.check_call([sys.executable, str(EX / "optimize_config.py"), str(perf), "-o", str(tuned)], stdout=subprocess.DEVNULL)
    cfg = json.loads(tuned.read_text())
    assert cfg["rules"] and all(r["min_bytes"] < r["max_bytes"] for r in cfg["rules"])
    ar = [r for r in cfg["rules"] if r["op"] == int(Cmd.ALLREDUCE)]
    assert ar[0]["min_bytes"] == 0 and ar[-1]["max_bytes"] == 1 << 62
    # force a known answer, then check that the plugin applies the file
    cfg["rules"] = [{"op": int(Cmd.ALLREDUCE), "min_bytes": 0, "max_bytes": 100000, "alg": "HostAllReduceSoleRing"},
                    {"op": int(Cmd.ALLREDUCE), "min_bytes": 100000, "max_bytes": 1 << 62, "alg": "HostAllReduceSoleRHD"}]
    tuned.write_text(json.dumps(cfg))
    so = tmp_path / "libconfig_tuner.so"
    subprocess.check_call(["g++", "-shared", "-fPIC", "-std=c++17", f"-I{ROOT / 'csrc' / 'include'}", str(EX / "config_tuner.cc"), "-o", str(so)])
    try:
        os.environ["HCCL_ALG_TUNER_PLUGIN"] = str(so)
        os.environ["HCCL_ALG_CONFIG_FILE"] = str(tuned)
        lib.HcclReloadEnvConfig()
        comms = hb.Communicator.host_sim(4)
        small = comms[0].explain(Cmd.ALLREDUCE, 1000, DataType.FP32)
        large = comms[0].explain(Cmd.ALLREDUCE, 1 << 20, DataType.FP32)
        assert small.startswith("selected HostAllReduceSoleRing") and "[tuner]" in small, small
        assert large.startswith("selected HostAllReduceSoleRHD"), large
        assert "[tuner]" not in comms[0].explain(Cmd.ALLGATHER, 1000, DataType.FP32)       # no rule: the model decides
        for c in comms:
            c.destroy()
    finally:
        os.environ.pop("HCCL_ALG_TUNER_PLUGIN", None)
        os.environ.pop("HCCL_ALG_CONFIG_FILE", None)
        lib.HcclReloadEnvConfig()
