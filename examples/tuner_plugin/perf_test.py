"""Step 1 of the tuning workflow: time every algorithm the selector could run.

    python examples/tuner_plugin/perf_test.py --host-sim 8 --out perf.jsonl
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 examples/tuner_plugin/perf_test.py --out perf.jsonl

For every operator and message size the script lists the algorithms that pass the selector's filters, forces each of
them in turn through the config tuner plugin (HCCL_ALG_FORCE, a fresh communicator per algorithm because a tuner is
created per communicator) and writes one JSON line per measurement: {"op", "cmd", "bytes", "alg", "us"}.
``--host-sim N`` runs N ranks as host threads on the host engine (no GPU needed); without it the script expects to
run under torchrun with one GPU per rank and times the device engines with CUDA events (max over ranks).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

import hccl_b200 as hb  # noqa: E402
from hccl_b200._lib import lib  # noqa: E402
from hccl_b200.types import Cmd, DataType  # noqa: E402

OPS = {"all_reduce": Cmd.ALLREDUCE, "all_gather": Cmd.ALLGATHER, "reduce_scatter": Cmd.REDUCE_SCATTER, "broadcast": Cmd.BROADCAST}


def build_plugin(workdir: Path) -> Path:
    so = workdir / "libconfig_tuner.so"
    src = Path(__file__).resolve().parent / "config_tuner.cc"
    subprocess.check_call(["g++", "-shared", "-fPIC", "-std=c++17", f"-I{ROOT / 'csrc' / 'include'}", str(src), "-o", str(so)])
    return so


def viable_algorithms(explain_text: str):
    names = []
    for line in explain_text.splitlines()[1:]:
        name, _, rest = line.strip().partition(": ")
        if name and not rest.startswith("filtered"):
            names.append(name)
    return names


def elements(op: str, nbytes: int, n: int) -> int:
    """Per-call element count (fp32) for a message of `nbytes` as the selector counts it."""
    per_rank = op in ("all_gather", "reduce_scatter")
    return max(1, nbytes // 4 // (n if per_rank else 1))


def run_host(op: str, comms, count: int, iters: int) -> float:
    n = len(comms)
    ins = [np.ones(count * (n if op == "reduce_scatter" else 1), np.float32) for _ in range(n)]
    outs = [np.zeros(count * (n if op == "all_gather" else 1), np.float32) for _ in range(n)]

    def body(r):
        c = comms[r]
        for _ in range(iters):
            if op == "all_reduce":
                c.all_reduce(ins[r], outs[r])
            elif op == "all_gather":
                c.all_gather(ins[r], outs[r])
            elif op == "reduce_scatter":
                c.reduce_scatter(ins[r], outs[r])
            else:
                c.broadcast(outs[r], 0)

    def once():
        ts = [threading.Thread(target=body, args=(r,)) for r in range(n)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        return (time.perf_counter() - t0) / iters * 1e6

    once()                                    # warm-up: selection, first-call checks
    return min(once() for _ in range(3))


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--host-sim", type=int, default=0, help="run this many ranks as host threads on the host engine")
    ap.add_argument("--ops", default="all_reduce,all_gather,reduce_scatter,broadcast")
    ap.add_argument("--sizes", default="4096,65536,1048576,16777216", help="message sizes in bytes")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--out", default="perf.jsonl")
    args = ap.parse_args()
    sizes = [int(s) for s in args.sizes.split(",")]
    workdir = Path(tempfile.mkdtemp(prefix="hccl_tuner_"))
    os.environ["HCCL_ALG_TUNER_PLUGIN"] = str(build_plugin(workdir))
    os.environ.pop("HCCL_ALG_CONFIG_FILE", None)
    rows = []
    if not args.host_sim:
        print("device mode: launch under torchrun; see bench/sweep.py for the timing loop this mode shares", file=sys.stderr)
        return device_mode(args, sizes)
    n = args.host_sim
    for op in args.ops.split(","):
        for nbytes in sizes:
            os.environ.pop("HCCL_ALG_FORCE", None)
            lib.HcclReloadEnvConfig()
            probe = hb.Communicator.host_sim(n)
            names = viable_algorithms(probe[0].explain(OPS[op], elements(op, nbytes, n), DataType.FP32))
            for c in probe:
                c.destroy()
            for alg in names:
                os.environ["HCCL_ALG_FORCE"] = alg
                comms = hb.Communicator.host_sim(n)
                us = run_host(op, comms, elements(op, nbytes, n), args.iters)
                used = comms[0].last_algorithm()
                for c in comms:
                    c.destroy()
                if used != alg:
                    continue                  # the selector could not honour the request (engine tier, HCCL_ALGO)
                rows.append({"op": op, "cmd": int(OPS[op]), "bytes": nbytes, "alg": alg, "us": round(us, 2), "ranks": n})
                print(rows[-1], flush=True)
    os.environ.pop("HCCL_ALG_FORCE", None)
    with open(args.out, "w") as f:
        for r in rows:
            f.write(json.dumps(r) + "\n")
    return 0


def device_mode(args, sizes) -> int:
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rows = []
    for op in args.ops.split(","):
        for nbytes in sizes:
            count = elements(op, nbytes, world)
            os.environ.pop("HCCL_ALG_FORCE", None)
            lib.HcclReloadEnvConfig()
            probe = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=64))
            names = viable_algorithms(probe.explain(OPS[op], count, DataType.FP32))
            probe.destroy()
            for alg in names:
                os.environ["HCCL_ALG_FORCE"] = alg
                comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=64))
                x = torch.ones(count * (world if op == "reduce_scatter" else 1), device="cuda")
                y = torch.zeros(count * (world if op == "all_gather" else 1), device="cuda")
                call = {"all_reduce": lambda: comm.all_reduce(x, y), "all_gather": lambda: comm.all_gather(x, y),
                        "reduce_scatter": lambda: comm.reduce_scatter(x, y), "broadcast": lambda: comm.broadcast(y, 0)}[op]
                for _ in range(5):
                    call()
                torch.cuda.synchronize()
                dist.barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(args.iters):
                    call()
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1) / args.iters * 1e3], device="cuda", dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                used = comm.last_algorithm()
                comm.destroy()
                if used == alg and rank == 0:
                    rows.append({"op": op, "cmd": int(OPS[op]), "bytes": nbytes, "alg": alg, "us": round(float(t), 2), "ranks": world})
                    print(rows[-1], flush=True)
    if rank == 0:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
