"""Measurements behind the headline metric: collective bus bandwidth next to NCCL on a fixed ladder of message sizes,
the fused matmul + collective kernels next to NCCL + cuBLAS with their roofline fraction, and value checks of both at the
benchmark shapes.  Used by ``bench.py`` (its ``extras`` and ``check`` blocks) and by the sweep scripts under ``bench/``.

Conventions (nccl-tests): ``bytes`` is the full buffer for all_reduce, the total over all ranks for all_gather /
reduce_scatter / all_to_all_v; algBW = bytes / time; busBW = algBW * factor(op, n).  Every time is taken on the device
with CUDA events and is the maximum over ranks; every iteration is timed on its own so that the slowest one is reported
next to the mean.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

from .timing import bus_bandwidth_factor

DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}
LADDER = (8, 64 << 10, 4 << 20, 256 << 20, 4 << 30)


def measured_peaks():
    """(GEMM TFLOP/s burst, NVLink GB/s per direction) the roofline fractions are taken against: the figures measured
    on this pool when the file the driver writes is present, else the stated fallback."""
    burst, _, link, src = measured_peaks_all()
    return burst, link, src


def measured_peaks_all():
    """(burst TFLOP/s, sustained TFLOP/s, NVLink GB/s per direction, source)."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    burst, sustained, src = 1590.0, 1400.0, "fallback"
    try:
        with open(path) as f:
            d = json.load(f)
            burst, src = float(d["bf16_tflops"]), "measured"
            sustained = float(d.get("bf16_tflops_sustained", sustained))
    except (OSError, KeyError, ValueError):
        pass
    return burst, sustained, 770.0, src


def timed_each(fn, warm, iters, group=None, isolate=False):
    """-> (mean ms, max ms) over `iters` separately timed launches, each the maximum over ranks.  Back to back by
    default (what a training step sees: clocks settle at the power limit, a rank's wait for the slowest peer is part of
    its time); `isolate=True` drains the device and lines the ranks up before every launch (the kernel alone at burst
    clocks: the number a roofline against a burst-measured peak is about)."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    multi = dist.is_initialized() and dist.get_world_size(group) > 1
    if multi:
        dist.barrier(group)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for e0, e1 in evs:
        if isolate:
            torch.cuda.synchronize()
            if multi:
                dist.barrier(group)
                torch.cuda.synchronize()
        e0.record()
        fn()
        e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) for e0, e1 in evs], device="cuda", dtype=torch.float64)
    if multi:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.mean().item(), t.max().item()


def graph_replay_us(fn, calls=10, replays=5, group=None):
    """Device time of one call when `calls` of them are captured in a CUDA graph and replayed (no host launch cost
    between them): the max over ranks of the best replay, in microseconds; None when the capture fails."""
    try:
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(calls):
                fn()
        g.replay()
        torch.cuda.synchronize()
        multi = dist.is_initialized() and dist.get_world_size(group) > 1
        best = float("inf")
        for _ in range(replays):
            if multi:
                dist.barrier(group)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) * 1000.0 / calls)
        t = torch.tensor([best], device="cuda", dtype=torch.float64)
        if multi:
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
        del g
        return t.item()
    except Exception:                                  # noqa: BLE001  (a library that cannot be captured just has no figure)
        torch.cuda.synchronize()
        return None


def _v_counts(n, world, rank):
    """Uneven split of n elements for the AlltoAllV rows: the block this rank sends to peer q is (1 + ((rank + q) % 3) / 4)
    shares wide; the matrix is symmetric, so receive counts equal send counts."""
    w = [4 + (rank + q) % 3 for q in range(world)]
    unit = n // (6 * world)
    if unit == 0:
        c = [n // world] * world
    else:
        c = [unit * x for x in w]
    d = [0] * world
    for q in range(1, world):
        d[q] = d[q - 1] + c[q - 1]
    return c, d


def collective_ladder(comm, sizes=LADDER, dtypes=("bf16", "fp32"), ops=("all_reduce", "all_gather", "reduce_scatter", "all_to_all_v"),
                      warm=5, iters=20, with_plain=True, emit=None):
    """Rows {op, dtype, bytes, hccl_sym_us, hccl_us, nccl_us, busbw..., ratio...}; `hccl_sym` = buffers from
    ``comm.empty`` (read and written in place on the peers), `hccl` = ordinary tensors (staged through the slab)."""
    world, rank = comm.world_size, comm.rank
    rows = []
    for dname in dtypes:
        dt = DTYPES[dname]
        es = torch.empty((), dtype=dt).element_size()
        top = max(sizes)
        max_elems = (max(1, top // es) + world - 1) // world * world
        g = torch.Generator(device="cuda").manual_seed(1000 + rank)
        plain_in = torch.empty(max_elems, device="cuda", dtype=dt)
        step = 1 << 26
        for o in range(0, max_elems, step):          # filled piecewise: no fp32 temporary of the whole buffer
            m = min(step, max_elems - o)
            plain_in[o:o + m] = (torch.rand(m, device="cuda", generator=g) * 2 - 1).to(dt)
        plain_out = torch.empty(max_elems, device="cuda", dtype=dt)
        sym_in, sym_out = comm.empty((max_elems,), dt), comm.empty((max_elems,), dt)
        sym_in.copy_(plain_in)
        for op in ops:
            for size in sizes:
                n = max(1, size // es)
                if op != "all_reduce":
                    n = max(world, n // world * world)
                per = n // world
                nbytes = n * es
                big = nbytes > (64 << 20)
                w_, it_ = (2, max(3, iters // 5)) if big else (warm, iters)
                sc, sd = _v_counts(n, world, rank)

                def make(impl):
                    src = sym_in if impl == "hccl_sym" else plain_in
                    dst = sym_out if impl == "hccl_sym" else plain_out
                    if impl == "nccl":
                        if op == "all_reduce":
                            return lambda: dist.all_reduce(plain_out[:n])
                        if op == "all_gather":
                            return lambda: dist.all_gather_into_tensor(plain_out[:n], plain_in[:per])
                        if op == "reduce_scatter":
                            return lambda: dist.reduce_scatter_tensor(plain_out[:per], plain_in[:n])
                        return lambda: dist.all_to_all_single(plain_out[:sum(sc)], plain_in[:sum(sc)], sc, sc)
                    if op == "all_reduce":
                        return lambda: comm.all_reduce(src[:n], dst[:n])
                    if op == "all_gather":
                        return lambda: comm.all_gather(src[:per], dst[:n])
                    if op == "reduce_scatter":
                        return lambda: comm.reduce_scatter(src[:n], dst[:per])
                    return lambda: comm.all_to_all_v(src, sc, sd, dst, sc, sd)

                moved = (sum(sc) if op == "all_to_all_v" else n) * es
                f = bus_bandwidth_factor("all_to_all" if op == "all_to_all_v" else op, world)
                row = {"op": op, "dtype": dname, "bytes": moved, "n_gpus": world}
                for impl in (("hccl_sym", "hccl", "nccl") if with_plain else ("hccl_sym", "nccl")):
                    mean, worst = timed_each(make(impl), w_, it_)
                    row[impl + "_us"] = mean * 1000
                    row[impl + "_max_us"] = worst * 1000
                    row[impl + "_busbw_gbs"] = moved / (mean * 1e-3) / 1e9 * f
                    if impl != "nccl":
                        row[impl + "_alg"] = comm.last_algorithm()
                if nbytes <= (4 << 20):
                    # without the host: what the device needs per call (launch-bound calls otherwise measure Python)
                    row["hccl_sym_graph_us"] = graph_replay_us(make("hccl_sym"))
                    row["nccl_graph_us"] = graph_replay_us(make("nccl"))
                    if row["hccl_sym_graph_us"] and row["nccl_graph_us"]:
                        row["sym_vs_nccl_graph"] = row["nccl_graph_us"] / row["hccl_sym_graph_us"]
                row["sym_vs_nccl"] = row["nccl_us"] / row["hccl_sym_us"]
                if with_plain:
                    row["plain_vs_nccl"] = row["nccl_us"] / row["hccl_us"]
                rows.append(row)
                if emit is not None:
                    emit(row)
        del plain_in, plain_out
        comm.free(sym_in)
        comm.free(sym_out)
        torch.cuda.empty_cache()
    return rows


def _maxerr(got, want):
    return ((got.float() - want.float()).abs().max() / want.float().abs().max().clamp_min(1e-20)).item()


def collective_check(comm, nbytes=4 << 20):
    """Largest error, relative to the largest expected value, of AllReduce / AllGather / ReduceScatter / AlltoAllV
    (bf16 and fp32, symmetric and ordinary buffers) against an fp32 reference computed from NCCL-gathered inputs."""
    world, rank = comm.world_size, comm.rank
    out = {}
    for dname in ("bf16", "fp32"):
        dt = DTYPES[dname]
        es = torch.empty((), dtype=dt).element_size()
        n = nbytes // es // world * world
        per = n // world
        g = torch.Generator(device="cuda").manual_seed(77 + rank)
        x = (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dt)
        allx = torch.empty(world * n, device="cuda", dtype=dt)
        dist.all_gather_into_tensor(allx, x)
        allx = allx.view(world, n)
        total = allx.float().sum(0)
        sx, so = comm.empty((n,), dt), comm.empty((n,), dt)
        sx.copy_(x)
        y = torch.empty(n, device="cuda", dtype=dt)
        worst = {}
        for label, src, dst in (("sym", sx, so), ("plain", x, y)):
            comm.all_reduce(src, dst)
            worst[f"all_reduce_{label}"] = _maxerr(dst, total)
            comm.all_gather(src[:per], dst)
            worst[f"all_gather_{label}"] = _maxerr(dst, allx[:, :per].reshape(-1))
            comm.reduce_scatter(src, dst[:per])
            worst[f"reduce_scatter_{label}"] = _maxerr(dst[:per], total[rank * per:(rank + 1) * per])
            sc, sd = _v_counts(n, world, rank)
            dst.zero_()
            comm.all_to_all_v(src, sc, sd, dst, sc, sd)
            want = torch.zeros(n, device="cuda", dtype=dt)
            for q in range(world):
                qc, qd = _v_counts(n, world, q)
                want[sd[q]:sd[q] + sc[q]] = allx[q, qd[rank]:qd[rank] + qc[rank]]
            worst[f"all_to_all_v_{label}"] = _maxerr(dst[:sum(sc)], want[:sum(sc)])
        # in-place on symmetric memory (every rank reads what the others are about to overwrite unless the library orders it)
        so.copy_(x)
        comm.all_reduce(so)
        worst["all_reduce_sym_inplace"] = _maxerr(so, total)
        torch.cuda.synchronize()
        comm.free(sx)
        comm.free(so)
        for k, v in worst.items():
            out[f"{k}_{dname}"] = v
    t = torch.tensor(list(out.values()), device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return dict(zip(out.keys(), t.tolist()))


def mc2_headline(comm, m=8192, hidden=8192, ffn=28672, tp_shape=8, warm=3, iters=10, emit=None):
    """AllGather->Matmul and Matmul->ReduceScatter at the tensor-parallel shapes of the named configuration (the weight
    shard is the 1/8 shard whatever the number of GPUs launched), the decode-sized Matmul->AllReduce, each next to
    NCCL + cuBLAS, with the largest error of the fused results against an fp32 reference.  Roofline: the slower of
    2MNK / measured GEMM peak and (n - 1)/n of the gathered or scattered matrix over the measured NVLink rate."""
    from ..ops import mc2

    world, rank = comm.world_size, comm.rank
    peak_tflops, sustained_tflops, link_gbs, src = measured_peaks_all()
    rows = []

    def out_row(row):
        row["roofline_denominators"] = {"gemm_tflops": peak_tflops, "gemm_tflops_sustained": sustained_tflops, "nvlink_gbs_per_direction": link_gbs,
                                        "source": src}
        row["timing"] = ("fused_ms / nccl_cublas_ms: launches timed alone (device drained and ranks lined up before each), against the burst "
                         "GEMM peak; *_b2b_ms: the same launches back to back, against the sustained peak")
        rows.append(row)
        if emit is not None:
            emit(row)

    torch.manual_seed(7 + rank)
    M, H, F = m, hidden, ffn // tp_shape
    m_per = M // world
    # ---- AllGather -> Matmul (push form: symmetric gathered buffer, ordinary shard)
    a_shard = torch.randn(m_per, H, device="cuda").bfloat16()
    w = (torch.randn(F, H, device="cuda") * 0.02).bfloat16()
    out = torch.empty(M, F, device="cuda", dtype=torch.bfloat16)
    gathered = comm.empty((M, H), torch.bfloat16)
    ref_g = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    t_fused, t_fused_max = timed_each(lambda: mc2.all_gather_matmul(comm, a_shard, w, out=out, gathered=gathered), warm, iters, isolate=True)
    t_fused_b2b, _ = timed_each(lambda: mc2.all_gather_matmul(comm, a_shard, w, out=out, gathered=gathered), warm, iters)

    def base_ag():
        dist.all_gather_into_tensor(ref_g, a_shard)
        torch.matmul(ref_g, w.t(), out=out)

    mc2.all_gather_matmul(comm, a_shard, w, out=out, gathered=gathered)
    torch.cuda.synchronize()
    got = out.clone()
    t_base, _ = timed_each(base_ag, warm, iters, isolate=True)
    t_base_b2b, _ = timed_each(base_ag, warm, iters)
    want = ref_g.float() @ w.float().t()
    err = max(_maxerr(got, want), _maxerr(gathered, ref_g))
    fl = 2.0 * M * F * H
    link_ms = (world - 1) * m_per * H * 2 / (link_gbs * 1e6)
    roof = max(fl / (peak_tflops * 1e9), link_ms)
    roof_b2b = max(fl / (sustained_tflops * 1e9), link_ms)
    out_row({"case": "ag_matmul", "m": M, "n": F, "k": H, "n_gpus": world, "fused_ms": t_fused, "fused_max_ms": t_fused_max, "nccl_cublas_ms": t_base,
             "fused_tflops": fl / t_fused / 1e9, "nccl_cublas_tflops": fl / t_base / 1e9, "roofline_ms": roof, "fraction_of_roofline": roof / t_fused,
             "vs_nccl_cublas": t_base / t_fused, "fused_b2b_ms": t_fused_b2b, "nccl_cublas_b2b_ms": t_base_b2b,
             "fraction_of_sustained_roofline_b2b": roof_b2b / t_fused_b2b, "vs_nccl_cublas_b2b": t_base_b2b / t_fused_b2b, "max_rel_err": err})
    comm.free(gathered)
    del want, ref_g, got
    # ---- Matmul -> ReduceScatter
    a = torch.randn(M, F, device="cuda").bfloat16()
    w2 = (torch.randn(H, F, device="cuda") * 0.02).bfloat16()
    out2 = torch.empty(m_per, H, device="cuda", dtype=torch.bfloat16)
    full = torch.empty(M, H, device="cuda", dtype=torch.bfloat16)
    t_fused, t_fused_max = timed_each(lambda: mc2.matmul_reduce_scatter(comm, a, w2, out=out2), warm, iters, isolate=True)
    t_fused_b2b, _ = timed_each(lambda: mc2.matmul_reduce_scatter(comm, a, w2, out=out2), warm, iters)
    got = out2.clone()

    def base_rs():
        torch.matmul(a, w2.t(), out=full)
        dist.reduce_scatter_tensor(out2, full)

    t_base, _ = timed_each(base_rs, warm, iters, isolate=True)
    t_base_b2b, _ = timed_each(base_rs, warm, iters)
    part = (a.float() @ w2.float().t())
    dist.all_reduce(part)
    err = _maxerr(got, part[rank * m_per:(rank + 1) * m_per])
    fl = 2.0 * M * H * F
    link_ms = (world - 1) * m_per * H * 2 / (link_gbs * 1e6)
    roof = max(fl / (peak_tflops * 1e9), link_ms)
    roof_b2b = max(fl / (sustained_tflops * 1e9), link_ms)
    out_row({"case": "matmul_rs", "m": M, "n": H, "k": F, "n_gpus": world, "fused_ms": t_fused, "fused_max_ms": t_fused_max, "nccl_cublas_ms": t_base,
             "fused_tflops": fl / t_fused / 1e9, "nccl_cublas_tflops": fl / t_base / 1e9, "roofline_ms": roof, "fraction_of_roofline": roof / t_fused,
             "vs_nccl_cublas": t_base / t_fused, "fused_b2b_ms": t_fused_b2b, "nccl_cublas_b2b_ms": t_base_b2b,
             "fraction_of_sustained_roofline_b2b": roof_b2b / t_fused_b2b, "vs_nccl_cublas_b2b": t_base_b2b / t_fused_b2b, "max_rel_err": err})
    del part, full, got
    # ---- Matmul -> AllReduce, decode shapes
    K = H // tp_shape
    for md in (16, 64, 256):
        a = torch.randn(md, K, device="cuda").bfloat16()
        w3 = (torch.randn(H, K, device="cuda") * 0.02).bfloat16()
        o = torch.empty(md, H, device="cuda", dtype=torch.bfloat16)
        t_fused, t_fused_max = timed_each(lambda: mc2.matmul_all_reduce(comm, a, w3, out=o), 2 * warm, 3 * iters)
        got = o.clone()

        def base_ar():
            torch.matmul(a, w3.t(), out=o)
            dist.all_reduce(o)

        t_base, _ = timed_each(base_ar, 2 * warm, 3 * iters)
        part = a.float() @ w3.float().t()
        dist.all_reduce(part)
        out_row({"case": "matmul_ar", "m": md, "n": H, "k": K, "n_gpus": world, "fused_us": t_fused * 1000, "fused_max_us": t_fused_max * 1000,
                 "nccl_cublas_us": t_base * 1000, "vs_nccl_cublas": t_base / t_fused, "max_rel_err": _maxerr(got, part)})
    torch.cuda.empty_cache()
    return rows


def gemm_headline(warm=3, iters=10):
    """One GPU: the tcgen05 matmul kernel next to cuBLAS at the shard shapes and at 8192^3 (L2 flushed between launches)."""
    from ..ops import mc2

    peak_tflops, _, src = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    rows = []
    for (m, n, k, name) in ((8192, 3584, 8192, "up_proj_shard"), (8192, 8192, 3584, "down_proj_shard"), (8192, 8192, 8192, "square_8192")):
        a = torch.randn(m, k, device="cuda").bfloat16()
        w = (torch.randn(n, k, device="cuda") * 0.02).bfloat16()
        out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)

        def run(fn):
            ts = []
            for i in range(warm + iters):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                if i >= warm:
                    ts.append(e0.elapsed_time(e1))
            return sum(ts) / len(ts)

        t_ours = run(lambda: mc2.matmul(a, w, out=out))
        got = out.clone()
        t_cublas = run(lambda: torch.matmul(a, w.t(), out=out))
        fl = 2.0 * m * n * k
        rows.append({"case": "matmul", "name": name, "m": m, "n": n, "k": k, "hccl_ms": t_ours, "cublas_ms": t_cublas, "hccl_tflops": fl / t_ours / 1e9,
                     "cublas_tflops": fl / t_cublas / 1e9, "fraction_of_peak": fl / t_ours / 1e9 / peak_tflops, "peak_source": src,
                     "max_rel_err_vs_cublas": _maxerr(got, out)})
    return rows
