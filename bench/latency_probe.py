"""Latency split of the collectives against NCCL on the same box: eager device time, host time per call and
device-only time (CUDA-graph replay of 10 calls).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 --master-port 29521 \
        bench/latency_probe.py

Environment: SIZES (comma list of bytes, default 4096,262144,4194304,268435456), OPS (comma list), GRAPH=0 skips the
graph rows.  Per (op, size) one JSON row from rank 0: `<impl>_us` = CUDA-event time per call over 100 back-to-back
calls (10 above 8 MiB), `<impl>_host_us` = host time per call of the same loop, `<impl>_graph_us` = per-call time of a
replayed graph.  impl: sym (symmetric buffers), plain (torch tensors), nccl.  bf16, max over ranks.
"""
import os, sys, time, json
import torch, torch.distributed as dist
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import hccl_b200 as hb

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
torch.cuda.set_device(local)
dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local))
comm = hb.Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=256))
dt = torch.bfloat16
N = 1 << 27
sin, sout = comm.empty((N,), dt), comm.empty((N,), dt)
pin = torch.randn(N, device="cuda").to(dt); pout = torch.empty(N, device="cuda", dtype=dt)
sin.copy_(pin)
sizes = [int(s) for s in os.environ.get("SIZES", "4096,262144,4194304,268435456").split(",")]
ops = os.environ.get("OPS", "all_reduce,reduce_scatter,all_gather,broadcast,all_to_all").split(",")

def mk(op, impl, n):
    per = n // world
    if impl == "nccl":
        return {"all_reduce": lambda: dist.all_reduce(pout[:n]), "all_gather": lambda: dist.all_gather_into_tensor(pout[:n], pin[:per]),
                "reduce_scatter": lambda: dist.reduce_scatter_tensor(pout[:per], pin[:n]), "broadcast": lambda: dist.broadcast(pout[:n], 0),
                "all_to_all": lambda: dist.all_to_all_single(pout[:n], pin[:n])}[op]
    s, d = (sin, sout) if impl == "sym" else (pin, pout)
    a, b, c_, e = s[:n], d[:n], s[:per], d[:per]
    return {"all_reduce": lambda: comm.all_reduce(a, b), "all_gather": lambda: comm.all_gather(c_, b),
            "reduce_scatter": lambda: comm.reduce_scatter(a, e), "broadcast": lambda: comm.broadcast(b, 0),
            "all_to_all": lambda: comm.all_to_all(a, b)}[op]

def dev_time(fn, iters):
    for _ in range(5): fn()
    torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(iters): fn()
    e1.record()
    host = (time.perf_counter() - t0) / iters * 1e6
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters * 1e3, host], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()

def graph_time(fn, reps=10, replays=10):
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        fn(); st.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            for _ in range(reps): fn()
    torch.cuda.synchronize(); dist.barrier()
    g.replay(); torch.cuda.synchronize(); dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays): g.replay()
    e1.record(); torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / (reps * replays) * 1e3], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()

for op in ops:
    for size in sizes:
        n = size // 2 // world * world
        row = {"op": op, "bytes": n * 2, "mb": os.environ.get("HCCL_MAX_BLOCKS", "")}
        for impl in ("sym", "plain", "nccl"):
            iters = 100 if size <= (8 << 20) else 10
            d, h = dev_time(mk(op, impl, n), iters)
            row[impl + "_us"] = round(d, 1); row[impl + "_host_us"] = round(h, 1)
            if impl != "plain" and os.environ.get("GRAPH", "1") == "1":
                try:
                    row[impl + "_graph_us"] = round(graph_time(mk(op, impl, n), 10 if size <= (8 << 20) else 2, 5), 1)
                except Exception as ex:
                    row[impl + "_graph_us"] = str(ex)[:60]
            if impl != "nccl": row[impl + "_alg"] = comm.last_algorithm()
        if rank == 0: print(json.dumps(row), flush=True)
comm.destroy(); dist.destroy_process_group()
