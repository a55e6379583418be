"""Step 2 of the tuning workflow: turn measurements into a configuration file for the config tuner plugin.

    python examples/tuner_plugin/optimize_config.py perf.jsonl -o tuned.json

Input: the JSON lines of perf_test.py.  For every operator the fastest algorithm at each measured size is kept and
neighbouring sizes with the same winner are merged into one rule; a rule covers the sizes from the geometric mean with
the previous measured size up to the geometric mean with the next one (the first rule starts at 0, the last one is
open-ended).  Output: {"rules": [{"op", "min_bytes", "max_bytes", "alg", "us"}]}.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from collections import defaultdict

OPEN_END = 1 << 62


def optimise(rows):
    best = defaultdict(dict)                 # cmd -> bytes -> (us, alg)
    for r in rows:
        cur = best[r["cmd"]].get(r["bytes"])
        if cur is None or r["us"] < cur[0]:
            best[r["cmd"]][r["bytes"]] = (r["us"], r["alg"])
    rules = []
    for cmd in sorted(best):
        sizes = sorted(best[cmd])
        for i, s in enumerate(sizes):
            lo = 0 if i == 0 else int(math.sqrt(sizes[i - 1] * s))
            hi = OPEN_END if i == len(sizes) - 1 else int(math.sqrt(s * sizes[i + 1]))
            us, alg = best[cmd][s]
            if rules and rules[-1]["op"] == cmd and rules[-1]["alg"] == alg and rules[-1]["max_bytes"] == lo:
                rules[-1]["max_bytes"] = hi
            else:
                rules.append({"op": cmd, "min_bytes": lo, "max_bytes": hi, "alg": alg, "us": us})
    return {"rules": rules}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("perf", help="JSON lines written by perf_test.py")
    ap.add_argument("-o", "--out", default="tuned.json")
    args = ap.parse_args()
    with open(args.perf) as f:
        rows = [json.loads(line) for line in f if line.strip()]
    if not rows:
        print("no measurements in " + args.perf, file=sys.stderr)
        return 1
    cfg = optimise(rows)
    with open(args.out, "w") as f:
        json.dump(cfg, f, indent=1)
    for r in cfg["rules"]:
        print(f"op {r['op']:>2}  [{r['min_bytes']:>12}, {r['max_bytes']:>20})  {r['alg']}  ({r['us']} us)")
    return 0


if __name__ == "__main__":
    sys.exit(main())
