"""Runs the tcgen05 matmul a few times on one shape (for profiling one kernel in isolation).

    python bench/gemm_one.py --m 4096 --n 4096 --k 4096 --iters 3
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hccl_b200.ops import mc2  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--m", type=int, default=4096)
ap.add_argument("--n", type=int, default=4096)
ap.add_argument("--k", type=int, default=4096)
ap.add_argument("--iters", type=int, default=3)
ap.add_argument("--cublas", action="store_true", help="run torch.matmul instead (comparison)")
args = ap.parse_args()
a = torch.randn(args.m, args.k, device="cuda").bfloat16()
w = (torch.randn(args.n, args.k, device="cuda") * 0.02).bfloat16()
out = torch.empty(args.m, args.n, device="cuda", dtype=torch.bfloat16)
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
for i in range(args.iters):
    e0.record()
    if args.cublas:
        torch.matmul(a, w.t(), out=out)
    else:
        mc2.matmul(a, w, out=out)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    print(f"iter {i}: {ms:.4f} ms, {2.0 * args.m * args.n * args.k / ms / 1e9:.1f} TFLOP/s")
