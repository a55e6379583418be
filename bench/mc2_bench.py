"""MC2 fused matmul + collective kernels against NCCL + cuBLAS at the same shapes.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29512 \
        bench/mc2_bench.py --out mc2_8gpu.jsonl

Shapes (tensor parallel over the N launched GPUs, bf16, weights N(0, 0.02), activations N(0, 1)):
  AllGather->Matmul      gathered activations [8192, 8192] x weight shard [8192, 28672 / 8]
  Matmul->ReduceScatter  [8192, 28672 / 8] x [28672 / 8, 8192], scattered over rows
  Matmul->AllReduce      M in {16, 64, 256}, K = 8192 / 8, N = 8192
and the plain tcgen05 matmul against torch.matmul (cuBLAS) for context.  Device-timed (CUDA events), max over ranks,
L2 flushed between timed iterations of the single-kernel cases.  TFLOPS counts the matmul only (2 M N K per rank).
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
from hccl_b200.ops import mc2  # noqa: E402


def timed(fn, warm=5, iters=20, flush=None):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    t = torch.tensor([total / iters], device="cuda", dtype=torch.float64)
    if dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def headline_rows(args):
    from hccl_b200.utils import headline

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
    comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
    rows = headline.mc2_headline(comm, m=args.m, hidden=args.hidden, ffn=args.ffn, tp_shape=args.tp_shape)
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
        if args.out:
            with open(args.out, "w") as f:
                for r in rows:
                    f.write(json.dumps(r) + "\n")
    comm.destroy()
    dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--tp-shape", type=int, default=8, help="the TP degree the shard shapes are cut for (8 in the named config)")
    ap.add_argument("--headline", action="store_true",
                    help="print the rows bench.py reports in its extras instead (hccl_b200.utils.headline.mc2_headline at --m / --tp-shape: every launch timed "
                         "alone AND back to back, roofline fractions against the burst and the sustained GEMM peak, errors against fp32)")
    args = ap.parse_args()
    if args.headline:
        return headline_rows(args)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    rows = []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    torch.manual_seed(7 + rank)
    M, H, F = args.m, args.hidden, args.ffn // args.tp_shape
    # ---- plain matmul vs cuBLAS (one GPU's share of the TP shapes)
    for (m, n, k, name) in ((M, F, H, "up_proj_shard"), (M, H, F, "down_proj_shard"), (8192, 8192, 8192, "square_8192")):
        a = torch.randn(m, k, device="cuda").bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
        t_ours = timed(lambda: mc2.matmul(a, w, out=out), flush=flush)
        t_cublas = timed(lambda: torch.matmul(a, w.t(), out=out), flush=flush)
        fl = 2.0 * m * n * k
        emit({"case": "matmul", "name": name, "m": m, "n": n, "k": k, "hccl_ms": t_ours, "cublas_ms": t_cublas, "hccl_tflops": fl / t_ours / 1e9,
              "cublas_tflops": fl / t_cublas / 1e9})
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
        comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
        m_per = M // world
        # ---- AllGather -> Matmul
        a_shard = comm.empty((m_per, H), torch.bfloat16)
        a_shard.copy_(torch.randn(m_per, H, device="cuda").bfloat16())
        w = (torch.randn(F, H, device="cuda") * 0.02).bfloat16()
        out = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
        gathered = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
        t_pull = timed(lambda: mc2.all_gather_matmul(comm, a_shard, w, out=out, gathered=gathered))
        # push form (the default of the TP layers): the gathered buffer is symmetric, the shard a plain tensor
        gathered_sym = comm.empty((M, H), torch.bfloat16)
        a_plain = a_shard.clone()
        t_fused = timed(lambda: mc2.all_gather_matmul(comm, a_plain, w, out=out, gathered=gathered_sym))

        def base_ag():
            dist.all_gather_into_tensor(gathered, a_shard)
            torch.matmul(gathered, w.t(), out=out)

        t_base = timed(base_ag)
        t_mm = timed(lambda: torch.matmul(gathered, w.t(), out=out))
        fl = 2.0 * M * F * H
        link_bytes = (world - 1) * m_per * H * 2
        roof_ms = max(fl / 1663.3e9, link_bytes / 770e6)       # measured burst GEMM peak and measured peer-copy bandwidth
        emit({"case": "ag_matmul", "m": M, "n": F, "k": H, "n_gpus": world, "fused_ms": t_fused, "fused_pull_ms": t_pull, "nccl_cublas_ms": t_base, "cublas_only_ms": t_mm,
              "fused_tflops": fl / t_fused / 1e9, "nccl_cublas_tflops": fl / t_base / 1e9, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / t_fused})
        # ---- Matmul -> ReduceScatter
        a = torch.randn(M, F, device="cuda").bfloat16()
        w2 = (torch.randn(H, F, device="cuda") * 0.02).bfloat16()
        out2 = torch.empty(m_per, H, device="cuda", dtype=torch.bfloat16)
        full = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
        t_fused = timed(lambda: mc2.matmul_reduce_scatter(comm, a, w2, out=out2))

        def base_rs():
            torch.matmul(a, w2.t(), out=full)
            dist.reduce_scatter_tensor(out2, full)

        t_base = timed(base_rs)
        fl = 2.0 * M * H * F
        link_bytes = (world - 1) * m_per * H * 2
        roof_ms = max(fl / 1663.3e9, link_bytes / 770e6)
        emit({"case": "matmul_rs", "m": M, "n": H, "k": F, "n_gpus": world, "fused_ms": t_fused, "nccl_cublas_ms": t_base,
              "fused_tflops": fl / t_fused / 1e9, "nccl_cublas_tflops": fl / t_base / 1e9, "roofline_ms": roof_ms, "fraction_of_roofline": roof_ms / t_fused})
        # ---- Matmul -> AllReduce, decode shapes
        K = H // args.tp_shape
        for m in (16, 64, 256):
            a = torch.randn(m, K, device="cuda").bfloat16()
            w3 = (torch.randn(H, K, device="cuda") * 0.02).bfloat16()
            o = torch.empty(m, H, device="cuda", dtype=torch.bfloat16)
            t_fused = timed(lambda: mc2.matmul_all_reduce(comm, a, w3, out=o), warm=10, iters=50)

            def base_ar():
                torch.matmul(a, w3.t(), out=o)
                dist.all_reduce(o)

            t_base = timed(base_ar, warm=10, iters=50)
            fl = 2.0 * m * H * K
            emit({"case": "matmul_ar", "m": m, "n": H, "k": K, "n_gpus": world, "fused_us": t_fused * 1000, "nccl_cublas_us": t_base * 1000,
                  "fused_tflops": fl / t_fused / 1e9, "nccl_cublas_tflops": fl / t_base / 1e9})
        comm.destroy()
        dist.destroy_process_group()
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
