"""Turns collective sweeps into the measurement file the selector's cost model loads
(``hccl_b200/data/link_model.json``, or the file ``HCCL_LINK_MODEL_FILE`` names).

    python bench/link_model.py sweep_2gpu.jsonl sweep_4gpu.jsonl sweep_8gpu.jsonl --out hccl_b200/data/link_model.json

Input rows are those of ``bench/sweep.py`` (``op, bytes, impl, time_us, n_gpus, alg``) or of the ``extras`` block of
``bench.py`` (``op, bytes, hccl_sym_us, hccl_sym_alg, n_gpus``).  Per GPU count the file gets one utilisation curve per
link class, keyed by the bytes one rank moves over one peer link:

* ``p2p``: from the pull AllGather on symmetric buffers, whose cost model is ``(p - 1) / p * bytes / (p2pGBs * util)``
  plus two barriers: ``util = ideal transfer time / (measured time - fixed cost)``;
* ``nvls``: from the switch AllReduce, ``(1 + 1 / p) * bytes / (nvlsGBs * util)``.

The reference keeps the same kind of table per link class and engine (cost_table.cc:437-457); there the tables are
typed into the source, here they come from a run on the box.
"""
from __future__ import annotations

import argparse
import json
from collections import defaultdict

P2P_GBS, NVLS_GBS = 770.0, 900.0
LAUNCH_US, BARRIER_US = 2.5, 2.2


def rows_of(path):
    out = []
    for line in open(path):
        line = line.strip()
        if not line.startswith("{"):
            continue
        r = json.loads(line)
        if "extras" in r:                                   # a bench.py line
            for x in r["extras"].get("collectives_busbw_vs_nccl", []):
                out.append({"op": x["op"], "bytes": x["bytes"], "n_gpus": x["n_gpus"], "dtype": x["dtype"], "time_us": x["hccl_sym_us"],
                            "alg": x.get("hccl_sym_alg", ""), "impl": "hccl_sym"})
        elif "impl" in r and "time_us" in r:
            out.append(r)
    return out


def build(paths):
    p2p, nvls = defaultdict(dict), defaultdict(dict)
    for path in paths:
        for r in rows_of(path):
            if r.get("impl") != "hccl_sym" or r.get("dtype", "bf16") != "bf16":
                continue
            p, nbytes, t = int(r["n_gpus"]), float(r["bytes"]), float(r["time_us"])
            fixed = LAUNCH_US + 2 * BARRIER_US
            if t <= fixed * 1.05:
                continue
            if r["op"] == "all_gather" and r.get("alg", "").startswith("P2pAllGatherSoleMesh") and "LL" not in r.get("alg", ""):
                ideal = (p - 1) / p * nbytes / (P2P_GBS * 1e3)
                p2p[p][nbytes / p] = max(1e-3, min(1.2, ideal / (t - fixed)))
            if r["op"] == "all_reduce" and r.get("alg", "").startswith("Nvls"):
                ideal = (1 + 1 / p) * nbytes / (NVLS_GBS * 1e3)
                nvls[p][nbytes / p] = max(1e-3, min(1.2, ideal / (t - fixed)))

    def curve(d):
        pts, best = [], 0.0
        for b in sorted(d):
            best = max(best, d[b])                          # a curve that dips is measurement noise: keep it monotone
            pts.append([b, round(best, 4)])
        return pts

    return {"gpu": "NVIDIA B200, NVLink 5 / NVSwitch", "source": "bench/link_model.py from " + ", ".join(paths),
            "link": {"p2pGBs": P2P_GBS, "nvlsGBs": NVLS_GBS, "launchUs": LAUNCH_US, "barrierUs": BARRIER_US},
            "utilisation": {"p2p": {str(p): curve(d) for p, d in sorted(p2p.items()) if d},
                            "nvls": {str(p): curve(d) for p, d in sorted(nvls.items()) if d}}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("inputs", nargs="+")
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    model = build(args.inputs)
    with open(args.out, "w") as f:
        json.dump(model, f, indent=1)
        f.write("\n")
    for kind, per in model["utilisation"].items():
        for p, pts in per.items():
            print(f"{kind} {p} GPUs: {len(pts)} points, top utilisation {pts[-1][1] if pts else None}")


if __name__ == "__main__":
    main()
