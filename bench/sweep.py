"""Collective bandwidth sweep against NCCL on the same box (nccl-tests conventions).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        bench/sweep.py --ops all_reduce,all_gather,reduce_scatter,broadcast,all_to_all --dtypes bf16,fp32 \
        --min-bytes 8 --max-bytes 1073741824 --out sweep_8gpu.jsonl

Per (op, dtype, size): 20 warm-up + 100 timed iterations (fewer above 64 MiB), every iteration timed on its own with
CUDA events (max over ranks), repeated `--repeats` times: `time_us` is the median of the repeats' means, `max_us` the
slowest single iteration of all repeats (an intermittent stall shows there, not in a footnote).  algBW = bytes / time,
busBW = algBW * factor.  `size` is the per-rank message size as in nccl-tests: the full buffer for all_reduce /
broadcast, the total (all ranks) for all_gather / reduce_scatter / all_to_all(_v).  Inputs are uniform[-1, 1] seeded
by rank.  Rows: impl in {hccl (plain buffers), hccl_sym (symmetric memory, zero copy), nccl}.  `all_to_all_v` moves
uneven blocks (4 : 5 : 6 shares, a symmetric count matrix).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import hccl_b200 as hb  # noqa: E402
from hccl_b200.utils import bus_bandwidth_factor  # noqa: E402
from hccl_b200.utils.headline import _v_counts, timed_each  # noqa: E402

DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


def timed(fn, warm, iters):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def human(b):
    for unit, size in (("GiB", 1 << 30), ("MiB", 1 << 20), ("KiB", 1 << 10)):
        if b >= size and b % size == 0:
            return f"{b // size} {unit}"
    return f"{b} B"


def write_markdown(rows, path, command, ladder=False):
    """One table per (op, dtype): time (busBW) of the symmetric-buffer and the ordinary-buffer path and of NCCL, the
    slowest single iteration of this library's symmetric path, the algorithm that ran, and the ratios.  `ladder`
    keeps every fourth size (8 B, 128 B, ... 4 GiB; for AlltoAllV the sizes nearest to those)."""
    import collections

    t = collections.OrderedDict()
    for r in rows:
        t.setdefault((r["op"], r["dtype"], r["bytes"]), {})[r["impl"]] = r
    if ladder:
        per_op = collections.OrderedDict()
        for (op, dt, b) in t:
            per_op.setdefault((op, dt), []).append(b)
        keep = set()
        for (op, dt), sizes in per_op.items():
            sizes = sorted(sizes)
            for i, b in enumerate(sizes):
                if i % 4 == 0 or i == len(sizes) - 1:
                    keep.add((op, dt, b))
        t = collections.OrderedDict((k, v) for k, v in t.items() if k in keep)
    world = rows[0]["n_gpus"] if rows else 0
    with open(path, "w") as f:
        f.write(f"# Collective sweep against NCCL, {world} x B200\n\nCommand:\n\n    {command}\n\n"
                "Every iteration is timed on its own with CUDA events (maximum over ranks); `us` is the median over the repeats of the mean, "
                "`max` the slowest single iteration of all repeats; busBW follows nccl-tests.  `sym` = buffers from `HcclMemAlloc` "
                "(read and written in place on the peers), `plain` = ordinary tensors staged through the slab.\n")
        cur = None
        for (op, dt, b), d in t.items():
            if (op, dt) != cur:
                cur = (op, dt)
                f.write(f"\n### {op}, {dt}\n\n| size | sym us (busBW GB/s) | sym max us | algorithm | plain us | NCCL us (busBW) | NCCL max us | sym / NCCL | plain / NCCL |\n"
                        "|---|---|---|---|---|---|---|---|---|\n")
            s_, p_, n_ = d.get("hccl_sym"), d.get("hccl"), d.get("nccl")
            if not (s_ and n_):
                continue
            f.write(f"| {human(b)} | {s_['time_us']:.1f} ({s_['busbw_gbs']:.0f}) | {s_.get('max_us', 0):.1f} | {s_['alg']} | "
                    f"{p_['time_us']:.1f} | {n_['time_us']:.1f} ({n_['busbw_gbs']:.0f}) | {n_.get('max_us', 0):.1f} | "
                    f"{n_['time_us'] / s_['time_us']:.2f}x | {n_['time_us'] / p_['time_us']:.2f}x |\n" if p_ else
                    f"| {human(b)} | {s_['time_us']:.1f} ({s_['busbw_gbs']:.0f}) | {s_.get('max_us', 0):.1f} | {s_['alg']} | - | "
                    f"{n_['time_us']:.1f} ({n_['busbw_gbs']:.0f}) | {n_.get('max_us', 0):.1f} | {n_['time_us'] / s_['time_us']:.2f}x | - |\n")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="all_reduce,all_gather,reduce_scatter,broadcast,all_to_all")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--min-bytes", type=int, default=8)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--impls", default="hccl,hccl_sym,nccl")
    ap.add_argument("--out", default="")
    ap.add_argument("--iters", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--markdown", default="", help="also write the tables as markdown to this file")
    ap.add_argument("--check", action="store_true", help="verify results against NCCL at every size")
    ap.add_argument("--from-jsonl", default="", help="render --markdown from the rows of an earlier run instead of measuring (no GPU needed)")
    ap.add_argument("--ladder", action="store_true", help="--markdown keeps every fourth size")
    ap.add_argument("--command", default="", help="with --from-jsonl: the command that produced the rows, quoted in the markdown")
    args = ap.parse_args()
    if args.from_jsonl:
        rows = [json.loads(line) for line in open(args.from_jsonl) if line.startswith("{")]
        write_markdown(rows, args.markdown, args.command or "(see the jsonl)", ladder=args.ladder)
        return

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=512))
    impls = args.impls.split(",")
    rows = []
    sizes = []
    b = args.min_bytes
    while b <= args.max_bytes:
        sizes.append(b)
        b *= 2
    for op in args.ops.split(","):
        for dname in args.dtypes.split(","):
            dt = DTYPES[dname]
            es = torch.empty((), dtype=dt).element_size()
            # one allocation per (op, dtype) at the largest size, views for the smaller ones
            max_elems = max(1, args.max_bytes // es)
            max_elems = (max_elems + world - 1) // world * world
            g = torch.Generator(device="cuda").manual_seed(1000 + rank)
            plain_in = (torch.rand(max_elems, device="cuda", generator=g) * 2 - 1).to(dt)
            plain_out = torch.empty(max_elems, device="cuda", dtype=dt)
            sym_in = sym_out = None
            if "hccl_sym" in impls:
                sym_in = comm.empty((max_elems,), dt)
                sym_out = comm.empty((max_elems,), dt)
                sym_in.copy_(plain_in)
            for size in sizes:
                n = max(1, size // es)
                if op in ("all_gather", "reduce_scatter", "all_to_all", "all_to_all_v"):
                    if n < world:
                        continue
                    n = n // world * world
                per = n // world
                nbytes = n * es
                iters = args.iters if nbytes <= (64 << 20) else max(5, args.iters // 10)
                warm = args.warmup if nbytes <= (64 << 20) else 3

                sc, sd = _v_counts(n, world, rank)

                def make(impl):
                    src = sym_in if impl == "hccl_sym" else plain_in
                    dst = sym_out if impl == "hccl_sym" else plain_out
                    if op == "all_to_all_v":
                        if impl == "nccl":
                            return lambda: dist.all_to_all_single(plain_out[:sum(sc)], plain_in[:sum(sc)], sc, sc)
                        return lambda: comm.all_to_all_v(src, sc, sd, dst, sc, sd)
                    if impl == "nccl":
                        if op == "all_reduce":
                            return lambda: dist.all_reduce(plain_out[:n])
                        if op == "all_gather":
                            return lambda: dist.all_gather_into_tensor(plain_out[:n], plain_in[:per])
                        if op == "reduce_scatter":
                            return lambda: dist.reduce_scatter_tensor(plain_out[:per], plain_in[:n])
                        if op == "broadcast":
                            return lambda: dist.broadcast(plain_out[:n], 0)
                        return lambda: dist.all_to_all_single(plain_out[:n], plain_in[:n])
                    if op == "all_reduce":
                        return lambda: comm.all_reduce(src[:n], dst[:n])
                    if op == "all_gather":
                        return lambda: comm.all_gather(src[:per], dst[:n])
                    if op == "reduce_scatter":
                        return lambda: comm.reduce_scatter(src[:n], dst[:per])
                    if op == "broadcast":
                        return lambda: comm.broadcast(dst[:n], 0)
                    return lambda: comm.all_to_all(src[:n], dst[:n])

                if op == "all_to_all_v":
                    nbytes = sum(sc) * es
                if args.check and op not in ("broadcast", "all_to_all_v"):
                    ref = torch.empty_like(plain_out[:n])
                    if op == "all_reduce":
                        ref.copy_(plain_in[:n]); dist.all_reduce(ref)
                    elif op == "all_gather":
                        dist.all_gather_into_tensor(ref, plain_in[:per])
                    elif op == "reduce_scatter":
                        dist.reduce_scatter_tensor(ref[:per], plain_in[:n])
                    else:
                        dist.all_to_all_single(ref, plain_in[:n])
                    for impl in impls:
                        if impl == "nccl":
                            continue
                        make(impl)()
                        torch.cuda.synchronize()
                        got = (sym_out if impl == "hccl_sym" else plain_out)
                        m = per if op == "reduce_scatter" else n
                        tol = 3e-2 if dt != torch.float32 else 1e-4
                        if not torch.allclose(got[:m].float(), ref[:m].float(), rtol=tol, atol=tol * world):
                            raise SystemExit(f"rank {rank}: {impl} {op} {dname} size {nbytes} differs from NCCL")
                for impl in impls:
                    fn = make(impl)
                    means, worst = [], 0.0
                    for _ in range(max(1, args.repeats)):
                        mean, mx = timed_each(fn, warm, iters)
                        means.append(mean)
                        worst = max(worst, mx)
                    ms = sorted(means)[len(means) // 2]
                    alg = nbytes / (ms * 1e-3) / 1e9
                    row = {"op": op, "dtype": dname, "bytes": nbytes, "impl": impl, "time_us": ms * 1000, "max_us": worst * 1000, "algbw_gbs": alg,
                           "busbw_gbs": alg * bus_bandwidth_factor("all_to_all" if op == "all_to_all_v" else op, world), "n_gpus": world,
                           "alg": comm.last_algorithm() if impl != "nccl" else "nccl"}
                    rows.append(row)
                    if rank == 0:
                        print(json.dumps(row), flush=True)
            del plain_in, plain_out
            if sym_in is not None:
                comm.free(sym_in)
                comm.free(sym_out)
            torch.cuda.empty_cache()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    if rank == 0 and args.markdown:
        write_markdown(rows, args.markdown, f"python -m torch.distributed.run --nnodes=1 --nproc-per-node {world} --master-addr 127.0.0.1 " + " ".join(sys.argv),
                       ladder=args.ladder)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
