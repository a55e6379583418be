"""Flagship benchmark: tokens/s of a Llama-3-70B-shaped 8-layer decoder stack
(hidden 8192, 64 q heads, 8 kv heads, head 128, SwiGLU 28672, RMSNorm, RoPE
500000), seq 4096, micro-batch 1, bf16, forward + backward + optimizer step,
tensor parallel over N GPUs with sequence parallel.  Column-parallel
projections run as fused AllGather->Matmul kernels and row-parallel ones as
fused Matmul->ReduceScatter kernels of this library.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3

``--impl nccl`` runs the same model on torch.distributed (NCCL) + torch.matmul
(cuBLAS).  ``--impl reference`` reports that HCCL itself cannot run here.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="hccl", choices=["hccl", "nccl", "reference"])
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--tiny", action="store_true", help="small model for smoke runs (not a benchmark result)")
    ap.add_argument("--graph", default="auto", choices=["auto", "off"], help="capture the whole step in one CUDA graph (falls back to eager)")
    return ap.parse_args()


def main():
    args = parse()
    if args.impl == "reference":
        # HCCL is an Ascend/CANN library: its CMake build needs the CANN toolkit (find_cann_package(hcomm ...)) and its
        # device code is AscendC for dav-c310 / dav-920r1; there is no setup.py / pyproject to install and no CUDA path.
        print(json.dumps({"impl": "reference", "unavailable": "HCCL builds only against Ascend CANN (no pip-installable package, no CUDA/sm_100 "
                          "path); pip install of the reference tree fails: neither setup.py nor pyproject.toml"}))
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        print(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}", file=sys.stderr)
        return 2
    torch.cuda.set_device(local)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    if world > 1:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import hccl_b200 as hb
    from hccl_b200.models import LlamaConfig, LlamaStack
    from hccl_b200.parallel import TPContext
    from hccl_b200.ops import fused as fused_ops
    from hccl_b200.utils import ClockSampler

    comm = None
    if args.impl == "hccl" and world > 1:
        comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
    ctx = TPContext(comm=comm, group=None, impl=args.impl)
    cfg = LlamaConfig.tiny(2) if args.tiny else LlamaConfig.llama3_70b_8layers()
    cfg.n_layers = args.layers if not args.tiny else cfg.n_layers
    torch.manual_seed(1234 + rank)
    model = LlamaStack(cfg, ctx)
    if args.impl == "hccl":
        from hccl_b200.ops import FusedAdamW
        opt = FusedAdamW(model.parameters(), lr=1e-5)                  # this library's single-launch AdamW kernel (same update rule)
        opt_note = "AdamW(hccl_b200 FusedAdamW kernel)"
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-5, fused=True, capturable=True)
        opt_note = "AdamW(torch fused)"
    seq = args.seq

    # synthetic token ids, uniform over the vocabulary, one fresh pinned host batch per step
    g = torch.Generator().manual_seed(99)
    host_batches = [torch.randint(0, cfg.vocab, (seq,), generator=g, dtype=torch.int64).pin_memory() for _ in range(args.steps + args.warmup)]
    dev_tokens = torch.empty(seq, dtype=torch.int64, device="cuda")
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step_device(tokens):
        opt.zero_grad(set_to_none=True)
        loss = model.loss(tokens)
        loss.backward()
        opt.step()
        return loss

    # The whole step (forward, backward, optimizer) as ONE CUDA graph: at 8 GPUs the kernels are short and an eager
    # step is bound by launch gaps.  Captured after the eager warm-up (all symmetric buffers and library state exist);
    # every flag / epoch the fused kernels use lives in device memory, so a replay runs the same protocol again.
    graph, static_loss, graph_note, launches_per_step = None, None, "off", 0

    def capture():
        nonlocal graph, static_loss, graph_note, launches_per_step
        try:
            g_ = torch.cuda.CUDAGraph()
            opt.zero_grad(set_to_none=True)
            l0 = ctx.launches + fused_ops.LAUNCHES
            with torch.cuda.graph(g_):
                loss_ = model.loss(dev_tokens)
                loss_.backward()
                opt.step()
            launches_per_step = ctx.launches + fused_ops.LAUNCHES - l0
            graph, static_loss, graph_note = g_, loss_, "whole step captured"
        except Exception as ex:                      # noqa: BLE001  (any capture failure falls back to the eager step)
            torch.cuda.synchronize()
            graph, graph_note = None, f"capture failed, eager step: {type(ex).__name__}: {str(ex)[:120]}"

    def step_any(tokens_dev):
        """One step on tokens already on the device (graph replay when captured)."""
        if graph is not None:
            dev_tokens.copy_(tokens_dev, non_blocking=True)
            graph.replay()
            ctx.launches += launches_per_step
            return static_loss
        return step_device(tokens_dev)

    def step_e2e(i):
        if graph is not None:
            dev_tokens.copy_(host_batches[i], non_blocking=True)      # H2D of this step's inputs from pinned memory
            graph.replay()
            ctx.launches += launches_per_step
            loss = static_loss
        else:
            dev_tokens.copy_(host_batches[i], non_blocking=True)
            loss = step_device(dev_tokens)
        loss_host.copy_(loss.detach(), non_blocking=True)             # D2H of the step's result
        torch.cuda.current_stream().synchronize()
        return float(loss_host)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-timed run (inputs already on the device), max over ranks
    dev_inputs = [b.cuda() for b in host_batches]
    for i in range(args.warmup):
        step_device(dev_inputs[i])
    barrier()
    if args.graph != "off":
        capture()
        barrier()
        if graph is not None:
            for i in range(min(2, args.warmup)):                       # warm the replay path as well
                step_any(dev_inputs[i])
            barrier()
    launches0 = ctx.launches + fused_ops.LAUNCHES
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(gpu_index=local) as clocks:
        ev0.record()
        for i in range(args.steps):
            step_any(dev_inputs[args.warmup + i])
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = ctx.launches + fused_ops.LAUNCHES - launches0      # fused matmul (+collective) kernels and element-wise kernels of this library
    # ---- end-to-end through the public API: H2D of inputs + D2H of the loss every step
    barrier()
    t0 = time.perf_counter()
    last = 0.0
    for i in range(args.steps):
        last = step_e2e(args.warmup + i)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1000.0 / args.steps
    if world > 1:
        t = torch.tensor([ms, e2e_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()

    if rank == 0:
        tokens = seq                           # micro-batch 1: the whole job processes one sequence per step
        out = {
            "metric": "tokens_per_sec_fwd_bwd_llama3_70b_shape_8layers_tp_sp", "value": tokens / (ms / 1000.0), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids uniform over vocab 128256; random-init N(0,0.02) weights",
            "impl": args.impl,
            "config": {"model": "llama3-70b-shaped decoder stack" + (" (tiny smoke variant)" if args.tiny else ""), "layers": cfg.n_layers,
                       "hidden": cfg.hidden, "ffn": cfg.ffn, "heads": cfg.n_heads, "kv_heads": cfg.n_kv_heads, "global_batch": 1, "seq_len": seq,
                       "parallelism": f"tp{world}+sp", "optimizer": opt_note, "loss": "mean product of neighbouring features of the final hidden states",
                       "l2": "inputs larger than L2: >13 GB of weights stream through per step", "cuda_graph": graph_note},
            "clocks": clocks.summary(),
            "e2e": {"value": tokens / (e2e_ms / 1000.0), "unit": "tokens/s", "ms_per_step": e2e_ms, "h2d_bytes_per_step": seq * 8, "d2h_bytes_per_step": 4,
                    "last_loss": last},
            "gpu_launches": launches,
        }
        print(json.dumps(out))
    if comm is not None:
        comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
