"""Summary of a timeline written by the trace build of the fused matmul kernels.

    python hccl_b200/build.py --trace
    HCCL_B200_LIB=build/lib/libhccl_b200_trace.so HCCL_MC2_TRACE_FILE=/tmp/t <your multi-rank program>
    python bench/mc2_trace_summary.py /tmp/t [--ranks 0,3]

Every line of `/tmp/t.rank<r>.jsonl` is one CTA of one traced launch with the sixteen words of `TraceWord`
(`csrc/kernels/mc2_gemm.cuh`): absolute points in global-timer nanoseconds, durations in SM cycles.  Per launch and rank
this prints when the start barrier completed, when the first remote rows were ready, when producer / MMA issuer /
epilogue finished, and the median / minimum / maximum over the CTAs of the time each role spent waiting or copying -
which says whether a fused kernel is short of operands (rows that arrive late), of accumulators (a slow drain) or of
neither.
"""
from __future__ import annotations

import argparse
import glob
import json
import statistics as st

START_NS, GO_NS, PROD_READY_CLK, PROD_FIRST_REMOTE_NS, PROD_EMPTY_CLK, PROD_END_NS, MMA_FULL_CLK, MMA_TMEM_CLK = range(8)
MMA_END_NS, EPI_PUSH_CLK, PROD_TOTAL_CLK, EPI_DRAIN_CLK, EPI_FULL_CLK, EPI_END_NS, EPI_TAIL_CLK, TILES = range(8, 16)


def load(prefix):
    rows = {}
    for path in sorted(glob.glob(prefix + ".rank*.jsonl")):
        for line in open(path):
            d = json.loads(line)
            rows.setdefault((d["kind"], d["launch"], d["rank"]), []).append(d)
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("prefix")
    ap.add_argument("--ranks", default="", help="comma-separated ranks to print (default: all)")
    args = ap.parse_args()
    want = {int(r) for r in args.ranks.split(",") if r != ""}
    rows = load(args.prefix)
    for (kind, launch, rank) in sorted(rows):
        if want and rank not in want:
            continue
        ctas = rows[(kind, launch, rank)]
        starts = [c["w"][START_NS] for c in ctas if c["w"][START_NS]]
        if not starts:
            continue
        t0 = min(starts)
        head = ctas[0]
        rates = [c["w"][PROD_TOTAL_CLK] / max(1, c["w"][PROD_END_NS] - c["w"][START_NS]) for c in ctas if c["w"][PROD_END_NS] > c["w"][START_NS]]
        ghz = st.median(rates) if rates else 1.5

        def us(clk):
            return clk / ghz / 1000.0

        leaders = [c for c in ctas if c["cta"] % 2 == 0]          # the MMA issuer runs in the leader CTA of a pair
        print(f"{kind} launch {launch} rank {rank}: M={head['M']} N={head['N']} K={head['K']} bn={head['bn']}, {len(ctas)} CTAs, SM clock {ghz:.2f} GHz")
        go = head["w"][GO_NS]
        print(f"  CTAs start within {(max(starts) - t0) / 1e3:.1f} us; start barrier done at {((go - t0) / 1e3) if go else float('nan'):.1f} us")
        first = [(c["w"][PROD_FIRST_REMOTE_NS] - t0) / 1e3 for c in ctas if c["w"][PROD_FIRST_REMOTE_NS]]
        if first:
            print(f"  first remote rows ready: min {min(first):.1f} median {st.median(first):.1f} max {max(first):.1f} us")
        for name, idx, sel in (("producer end", PROD_END_NS, ctas), ("MMA issuer end", MMA_END_NS, leaders), ("epilogue end (with tail)", EPI_END_NS, ctas)):
            v = [(c["w"][idx] - t0) / 1e3 for c in sel if c["w"][idx]]
            if v:
                print(f"  {name:32s} median {st.median(v):7.1f}  max {max(v):7.1f} us")
        for name, idx, sel in (("producer waits for rows", PROD_READY_CLK, ctas), ("producer waits for free stages", PROD_EMPTY_CLK, ctas),
                               ("MMA waits for operands", MMA_FULL_CLK, leaders), ("MMA waits for an accumulator", MMA_TMEM_CLK, leaders),
                               ("epilogue copies / reduces", EPI_PUSH_CLK, ctas), ("epilogue waits for a tile", EPI_FULL_CLK, ctas),
                               ("epilogue drains", EPI_DRAIN_CLK, ctas), ("epilogue tail (after last tile)", EPI_TAIL_CLK, ctas)):
            v = [us(c["w"][idx]) for c in sel]
            print(f"  {name:32s} median {st.median(v):7.1f}  min {min(v):7.1f}  max {max(v):7.1f} us")
        tiles = [c["w"][TILES] for c in ctas]
        print(f"  tiles per CTA: {min(tiles)} - {max(tiles)}")


if __name__ == "__main__":
    main()
