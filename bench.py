"""Flagship benchmark: tokens/s of a Llama-3-70B-shaped 8-layer decoder stack
(hidden 8192, 64 q heads, 8 kv heads, head 128, SwiGLU 28672, RMSNorm, RoPE
500000), seq 4096, micro-batch 1, bf16, forward + backward + optimizer step,
tensor parallel over N GPUs with sequence parallel.  Column-parallel
projections run as fused AllGather->Matmul kernels and row-parallel ones as
fused Matmul->ReduceScatter kernels of this library.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 5 --warmup 3

One process runs, one after the other:
  * the library arm (fused matmul + collective kernels, this library's collectives);
  * the same-box baseline arm: the SAME model, element-wise kernels, optimizer kernel and whole-step CUDA graph, with
    torch.distributed (NCCL) collectives and torch.matmul (cuBLAS) in place of this library's.  ``vs_baseline`` is the
    end-to-end ratio of the two; the baseline's own line is kept under ``"baseline"``;
  * ``extras``: the headline metric itself - bus bandwidth of AllReduce / AllGather / ReduceScatter / AlltoAllV next to
    NCCL on a ladder of message sizes (bf16 and fp32), and the fused AllGather->Matmul / Matmul->ReduceScatter /
    Matmul->AllReduce kernels next to NCCL + cuBLAS with their roofline fractions (one GPU: the matmul kernel next to
    cuBLAS);
  * ``check``: largest errors of the collectives and of the fused kernels at the benchmark shapes against fp32
    references.
``--impl nccl`` runs the baseline arm alone, ``--impl reference`` reports that HCCL itself cannot run here,
``--no-extras`` skips the last two blocks.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import gc
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
    ap.add_argument("--no-extras", action="store_true", help="skip the bandwidth ladder, the fused-kernel table and the value checks")
    ap.add_argument("--no-baseline", action="store_true", help="skip the NCCL + cuBLAS arm")
    ap.add_argument("--ladder-max-bytes", type=int, default=4 << 30)
    return ap.parse_args()


def run_arm(impl, args, comm, cfg, rank, world, local, host_batches):
    """One arm of the model benchmark -> dict with device-timed and end-to-end figures."""
    import torch
    import torch.distributed as dist

    from hccl_b200.models import LlamaStack
    from hccl_b200.ops import FusedAdamW
    from hccl_b200.ops import fused as fused_ops
    from hccl_b200.parallel import TPContext
    from hccl_b200.utils import ClockSampler

    seq = args.seq
    # both arms: this library's element-wise kernels and optimizer kernel, whole step in one CUDA graph; they differ in
    # the matmul kernels and the collectives only
    ctx = TPContext(comm=comm if impl == "hccl" else None, group=None, impl=impl, fused_ops=True)
    torch.manual_seed(1234 + rank)
    model = LlamaStack(cfg, ctx)
    opt = FusedAdamW(model.parameters(), lr=1e-5)
    dev_tokens = torch.empty(seq, dtype=torch.int64, device="cuda")
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def step_device(tokens):
        opt.zero_grad(set_to_none=True)
        loss = model.loss(tokens)
        loss.backward()
        model.sync_replicated_grads()
        opt.step()
        total = loss.detach().clone()
        return ctx.all_reduce_(total, "loss")             # the ranks' shares add up to the loss of the whole sequence

    # The whole step (forward, backward, optimizer) as ONE CUDA graph: at 8 GPUs the kernels are short and an eager
    # step is bound by launch gaps.  Captured after the eager warm-up (all symmetric buffers and library state exist);
    # every flag / epoch the fused kernels use lives in device memory, so a replay runs the same protocol again.
    state = {"graph": None, "loss": None, "note": "off", "per_step": 0}

    def counted():
        return ctx.launches + fused_ops.LAUNCHES

    def capture():
        try:
            g_ = torch.cuda.CUDAGraph()
            opt.zero_grad(set_to_none=True)
            l0 = counted()
            with torch.cuda.graph(g_):
                loss_ = step_device(dev_tokens)
            state.update(graph=g_, loss=loss_, note="whole step captured", per_step=counted() - l0)
        except Exception as ex:                      # noqa: BLE001  (any capture failure falls back to the eager step)
            torch.cuda.synchronize()
            state.update(graph=None, note=f"capture failed, eager step: {type(ex).__name__}: {str(ex)[:120]}")

    def step_any(tokens_dev):
        """One step on tokens already on the device (graph replay when captured)."""
        if state["graph"] is not None:
            dev_tokens.copy_(tokens_dev, non_blocking=True)
            state["graph"].replay()
            ctx.launches += state["per_step"]
            return state["loss"]
        return step_device(tokens_dev)

    def step_e2e(i):
        dev_tokens.copy_(host_batches[i], non_blocking=True)          # H2D of this step's inputs from pinned memory
        if state["graph"] is not None:
            state["graph"].replay()
            ctx.launches += state["per_step"]
            loss = state["loss"]
        else:
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
        if state["graph"] is not None:
            for i in range(min(2, args.warmup)):                       # warm the replay path as well
                step_any(dev_inputs[i])
            barrier()
    launches0 = counted()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(gpu_index=local) as clocks:
        ev0.record()
        for i in range(args.steps):
            step_any(dev_inputs[args.warmup + i])
        ev1.record()
        barrier()
    ms = ev0.elapsed_time(ev1) / args.steps
    launches = counted() - launches0      # this library's kernels in the timed region: matmul (+collective), element-wise, optimizer, collectives
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
    res = {"impl": impl, "ms_per_step": ms, "tokens_per_s": seq / (ms / 1000.0), "e2e_ms_per_step": e2e_ms, "e2e_tokens_per_s": seq / (e2e_ms / 1000.0),
           "last_loss": last, "cuda_graph": state["note"], "gpu_launches": launches, "clocks": clocks.summary()}
    # give the memory back before the next arm
    state.update(graph=None, loss=None)
    del model, opt, dev_inputs
    ctx.release()
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    return res


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
    from hccl_b200.models import LlamaConfig
    from hccl_b200.utils import headline

    comm = None
    if world > 1:
        comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
    cfg = LlamaConfig.tiny(2) if args.tiny else LlamaConfig.llama3_70b_8layers()
    cfg.n_layers = args.layers if not args.tiny else cfg.n_layers
    seq = args.seq
    # synthetic token ids, uniform over the vocabulary, one fresh pinned host batch per step
    g = torch.Generator().manual_seed(99)
    host_batches = [torch.randint(0, cfg.vocab, (seq,), generator=g, dtype=torch.int64).pin_memory() for _ in range(args.steps + args.warmup)]

    main_arm = run_arm(args.impl, args, comm, cfg, rank, world, local, host_batches)
    base_arm = None
    if args.impl == "hccl" and not args.no_baseline:
        base_arm = run_arm("nccl", args, comm, cfg, rank, world, local, host_batches)

    extras, check = None, None
    if args.impl == "hccl" and not args.no_extras:
        t0 = time.perf_counter()
        extras, check = {}, {}

        def guarded(name, fn):
            """Runs one block of the extras; a failure on any rank ends that block on every rank (they agree over NCCL)
            and is reported in the output instead of taking the step measurement down with it."""
            res, err = None, None
            try:
                res = fn()
                torch.cuda.synchronize()
            except Exception as ex:                      # noqa: BLE001
                err = f"{type(ex).__name__}: {ex}"[:300]
            if world > 1:
                flag = torch.tensor([0 if err else 1], device="cuda", dtype=torch.int32)
                dist.all_reduce(flag, op=dist.ReduceOp.MIN)
                if int(flag.item()) == 0 and err is None:
                    err = "another rank failed in this block"
            if err is not None:
                extras.setdefault("errors", {})[name] = err
                return None
            return res

        if world > 1:
            sizes = tuple(s for s in headline.LADDER if s <= args.ladder_max_bytes)
            fused = guarded("fused_matmul_collective_vs_nccl_cublas", lambda: headline.mc2_headline(comm) if not args.tiny else [])
            extras["fused_matmul_collective_vs_nccl_cublas"] = fused
            check["fused_kernels_max_rel_err"] = {r["case"] + (f"_m{r['m']}" if r["case"] == "matmul_ar" else ""): r["max_rel_err"] for r in (fused or [])}
            ladder = []                                   # rows are kept as they come: a failure late in the ladder loses nothing before it
            guarded("collectives_busbw_vs_nccl", lambda: headline.collective_ladder(comm, sizes=sizes, emit=ladder.append))
            extras["collectives_busbw_vs_nccl"] = ladder
            check["collectives_max_rel_err"] = guarded("collectives_max_rel_err", lambda: headline.collective_check(comm))
        else:
            extras["matmul_vs_cublas"] = guarded("matmul_vs_cublas", headline.gemm_headline)
            check["matmul_max_rel_err_vs_cublas"] = {r["name"]: r["max_rel_err_vs_cublas"] for r in (extras["matmul_vs_cublas"] or [])}
        check["model_loss_library_vs_baseline"] = [main_arm["last_loss"], base_arm["last_loss"] if base_arm else None]
        extras["seconds"] = time.perf_counter() - t0

    if rank == 0:
        tokens = seq                           # micro-batch 1: the whole job processes one sequence per step
        out = {
            "metric": "tokens_per_sec_fwd_bwd_llama3_70b_shape_8layers_tp_sp", "value": main_arm["tokens_per_s"], "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_arm["ms_per_step"], "higher_is_better": True,
            "scaling": "strong",
            # same-box NCCL + cuBLAS arm under identical settings, end to end (the reference itself publishes no number for this metric)
            "vs_baseline": (main_arm["e2e_tokens_per_s"] / base_arm["e2e_tokens_per_s"]) if base_arm else None,
            "dtype": "bf16", "data": "synthetic token ids uniform over vocab 128256; random-init N(0,0.02) weights",
            "impl": args.impl,
            "config": {"model": "llama3-70b-shaped decoder stack" + (" (tiny smoke variant)" if args.tiny else ""), "layers": cfg.n_layers,
                       "hidden": cfg.hidden, "ffn": cfg.ffn, "heads": cfg.n_heads, "kv_heads": cfg.n_kv_heads, "global_batch": 1, "seq_len": seq,
                       "parallelism": f"tp{world}+sp", "optimizer": "AdamW(hccl_b200 FusedAdamW kernel), both arms",
                       "loss": "mean over the whole sequence of the product of neighbouring features of the final hidden states",
                       "embedding": "table cut along the hidden dimension, one AlltoAll to sequence shards" if world > 1 else "one table",
                       "replicated_grads": "RMSNorm weight gradients summed over the group every step",
                       "l2": "inputs larger than L2: >13 GB of weights stream through per step", "cuda_graph": main_arm["cuda_graph"]},
            "clocks": main_arm["clocks"],
            "e2e": {"value": main_arm["e2e_tokens_per_s"], "unit": "tokens/s", "ms_per_step": main_arm["e2e_ms_per_step"], "h2d_bytes_per_step": seq * 8,
                    "d2h_bytes_per_step": 4, "last_loss": main_arm["last_loss"]},
            "gpu_launches": main_arm["gpu_launches"],
        }
        if base_arm:
            out["baseline"] = {"what": "same model, element-wise kernels, optimizer kernel and CUDA graph; torch.distributed (NCCL) collectives + "
                                       "torch.matmul (cuBLAS)", "value": base_arm["tokens_per_s"], "ms_per_step": base_arm["ms_per_step"],
                               "e2e": {"value": base_arm["e2e_tokens_per_s"], "ms_per_step": base_arm["e2e_ms_per_step"], "last_loss": base_arm["last_loss"]},
                               "cuda_graph": base_arm["cuda_graph"], "clocks": base_arm["clocks"],
                               "device_timed_ratio": main_arm["tokens_per_s"] / base_arm["tokens_per_s"]}
        if extras is not None:
            out["extras"] = extras
            out["check"] = check
        print(json.dumps(out))
    if comm is not None:
        try:
            comm.destroy()
        except Exception:                                # noqa: BLE001  (a communicator that reported an error above)
            pass
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
