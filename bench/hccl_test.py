"""hccl_test-style command line: one operator over a range of sizes, with the columns of the reference's on-board
benchmark (``mpirun -n 8 ./bin/all_reduce_test -b 8K -e 64M -f 2 -d fp32 -o sum -p 8`` prints ``aveg_time``,
``alg_bandwidth`` and ``check_result``, docs/en/build/build.md:302-316).

    # 8 GPUs, one process per GPU
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/hccl_test.py --op all_reduce -b 8K -e 64M -f 2 -d fp32 -o sum
    # no GPU: ranks as host threads on the host engine
    python bench/hccl_test.py --op all_gather -b 1K -e 1M -f 4 -d fp16 -p 4 --host-sim

``-b`` / ``-e``: first and last message size in bytes (K, M, G suffixes), ``-f``: multiplication factor between sizes,
``-d``: data type, ``-o``: reduce operation, ``-p``: rank count (host engine only; on GPUs it is the world size),
``-n`` / ``-w``: timed and warm-up iterations, ``-c 0``: skip the result check.  The size is the per-rank message as in
nccl-tests (the whole buffer for all_reduce / broadcast / reduce, the total over ranks for all_gather /
reduce_scatter / alltoall).  Device runs are timed with CUDA events and the maximum over ranks is reported; the check
compares against a NumPy / PyTorch computation of the operator's definition on rank-dependent inputs.
"""
from __future__ import annotations

import argparse
import os
import sys
import threading
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import hccl_b200 as hb  # noqa: E402
from hccl_b200 import ReduceOp  # noqa: E402

OPS = ("all_reduce", "all_gather", "reduce_scatter", "broadcast", "reduce", "alltoall", "scatter")
NP_TYPES = {"fp32": np.float32, "fp16": np.float16, "fp64": np.float64, "int8": np.int8, "int32": np.int32, "int64": np.int64}
RED = {"sum": ReduceOp.SUM, "prod": ReduceOp.PROD, "max": ReduceOp.MAX, "min": ReduceOp.MIN}


def parse_size(text: str) -> int:
    mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}
    t = text.strip().upper()
    return int(float(t[:-1]) * mult[t[-1]]) if t[-1] in mult else int(t)


def sizes(args):
    s = parse_size(args.b)
    end = parse_size(args.e)
    while s <= end:
        yield s
        if args.f <= 1:
            break
        s = int(s * args.f)


def shapes(op: str, nbytes: int, esize: int, p: int):
    """(send elements, recv elements) per rank for a message of nbytes."""
    total = max(p, nbytes // esize // p * p)         # a multiple of the rank count
    per = total // p
    return {"all_reduce": (total, total), "broadcast": (total, total), "reduce": (total, total), "all_gather": (per, total),
            "reduce_scatter": (total, per), "alltoall": (total, total), "scatter": (total, per)}[op]


def host_input(rank: int, n: int, dtype):
    # small integers: sums and products are exact in every type, so the check can demand equality
    return ((np.arange(n) + rank) % 3 + 1).astype(dtype)


def expected(op: str, red: str, ins, rank: int, p: int, root: int):
    fold = {"sum": np.add, "prod": np.multiply, "max": np.maximum, "min": np.minimum}[red]
    if op in ("all_reduce", "reduce", "reduce_scatter"):
        acc = ins[0].copy()
        for x in ins[1:]:
            acc = fold(acc, x)
        if op == "reduce_scatter":
            per = acc.size // p
            return acc[rank * per:(rank + 1) * per]
        return acc if op == "all_reduce" or rank == root else None
    if op == "all_gather":
        return np.concatenate(ins)
    if op == "broadcast":
        return ins[root]
    if op == "scatter":
        per = ins[root].size // p
        return ins[root][rank * per:(rank + 1) * per]
    per = ins[0].size // p                                  # alltoall
    return np.concatenate([ins[q][rank * per:(rank + 1) * per] for q in range(p)])


def call(comm, op: str, red, send, recv, root: int):
    if op == "all_reduce":
        comm.all_reduce(send, recv, red)
    elif op == "all_gather":
        comm.all_gather(send, recv)
    elif op == "reduce_scatter":
        comm.reduce_scatter(send, recv, red)
    elif op == "broadcast":
        comm.broadcast(recv, root)
    elif op == "reduce":
        comm.reduce(send, recv, root, red)
    elif op == "scatter":
        comm.scatter(send, recv, root)
    else:
        comm.all_to_all(send, recv)


def run_host(args) -> int:
    p, dtype, root = args.p, NP_TYPES[args.d], 0
    comms = hb.Communicator.host_sim(p, None, hb.make_config(buffer_mib=max(64, 4 * parse_size(args.e) >> 20)))
    print(f"# host engine, {p} ranks as threads; op {args.op} dtype {args.d} reduce {args.o}")
    print(f"{'data_size(B)':>14} {'aveg_time(us)':>14} {'alg_bandwidth(GB/s)':>20} {'check_result':>13}")
    bad = 0
    for nbytes in sizes(args):
        ns, nr = shapes(args.op, nbytes, np.dtype(dtype).itemsize, p)
        ins = [host_input(r, ns, dtype) for r in range(p)]
        outs = [np.zeros(nr, dtype) for _ in range(p)]
        if args.op == "broadcast":
            outs = [ins[r].copy() for r in range(p)]

        def body(r, iters):
            for _ in range(iters):
                call(comms[r], args.op, RED[args.o], ins[r], outs[r], root)

        def timed(iters):
            ts = [threading.Thread(target=body, args=(r, iters)) for r in range(p)]
            t0 = time.perf_counter()
            [t.start() for t in ts]
            [t.join() for t in ts]
            return (time.perf_counter() - t0) / iters

        timed(args.w)
        sec = timed(args.n)
        ok = True
        if args.c:
            for r in range(p):
                want = expected(args.op, args.o, ins, r, p, root)
                ok = ok and (want is None or np.array_equal(outs[r], want))
        bad += 0 if ok else 1
        print(f"{nbytes:>14} {sec * 1e6:>14.2f} {nbytes / sec / 1e9:>20.3f} {('success' if ok else 'FAILED') if args.c else 'skipped':>13}", flush=True)
    for c in comms:
        c.destroy()
    return 1 if bad else 0


def run_device(args) -> int:
    import torch
    import torch.distributed as dist

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
    tdt = {"fp32": torch.float32, "fp16": torch.float16, "fp64": torch.float64, "int8": torch.int8, "int32": torch.int32, "int64": torch.int64,
           "bf16": torch.bfloat16}[args.d]
    npdt = NP_TYPES.get(args.d, np.float32)
    root, bad = 0, 0
    if rank == 0:
        print(f"# {world} GPUs; op {args.op} dtype {args.d} reduce {args.o}")
        print(f"{'data_size(B)':>14} {'aveg_time(us)':>14} {'alg_bandwidth(GB/s)':>20} {'check_result':>13}")
    for nbytes in sizes(args):
        ns, nr = shapes(args.op, nbytes, torch.empty(0, dtype=tdt).element_size(), world)
        ins = [host_input(r, ns, npdt) for r in range(world)] if args.c else None
        send = (torch.from_numpy(ins[rank]).cuda() if args.c else torch.ones(ns, device="cuda")).to(tdt)
        recv = send.clone() if args.op == "broadcast" else torch.zeros(nr, dtype=tdt, device="cuda")
        for _ in range(args.w):
            call(comm, args.op, RED[args.o], send, recv, root)
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.n):
            call(comm, args.op, RED[args.o], send, recv, root)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.n * 1e-3], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ok = torch.ones(1, device="cuda")
        if args.c and args.op != "broadcast":        # a repeated in-place broadcast keeps the root's data: checked like the rest
            want = expected(args.op, args.o, ins, rank, world, root)
            if want is not None and not np.array_equal(recv.float().cpu().numpy(), want.astype(np.float32)):
                ok.zero_()
        elif args.c:
            if not np.array_equal(recv.float().cpu().numpy(), ins[root].astype(np.float32)):
                ok.zero_()
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        good = bool(ok.item())
        bad += 0 if good else 1
        if rank == 0:
            sec = float(t)
            print(f"{nbytes:>14} {sec * 1e6:>14.2f} {nbytes / sec / 1e9:>20.3f} {('success' if good else 'FAILED') if args.c else 'skipped':>13}", flush=True)
    comm.destroy()
    dist.destroy_process_group()
    return 1 if bad else 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=OPS, default="all_reduce")
    ap.add_argument("-b", default="8K")
    ap.add_argument("-e", default="64M")
    ap.add_argument("-f", type=float, default=2.0)
    ap.add_argument("-d", default="fp32")
    ap.add_argument("-o", default="sum", choices=sorted(RED))
    ap.add_argument("-p", type=int, default=8)
    ap.add_argument("-n", type=int, default=20)
    ap.add_argument("-w", type=int, default=5)
    ap.add_argument("-c", type=int, default=1)
    ap.add_argument("--host-sim", action="store_true")
    args = ap.parse_args()
    if args.host_sim:
        if args.d not in NP_TYPES:
            print(f"host engine: data type {args.d} is not available in NumPy", file=sys.stderr)
            return 2
        return run_host(args)
    if "RANK" not in os.environ:
        print("launch under torch.distributed.run (one process per GPU), or pass --host-sim", file=sys.stderr)
        return 2
    return run_device(args)


if __name__ == "__main__":
    sys.exit(main())
