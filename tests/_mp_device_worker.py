"""One rank of a multi-process device test: python _mp_device_worker.py <rank> <world> <rendezvous-file> <scenario>."""
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch

import hccl_b200 as hb
from hccl_b200 import Communicator, ReduceOp


def rendezvous(rank, path):
    if rank == 0:
        info = Communicator.get_root_info()
        tmp = path + ".tmp"
        with open(tmp, "wb") as f:
            f.write(info)
        os.replace(tmp, path)
        return info
    t0 = time.time()
    while not os.path.exists(path):
        if time.time() - t0 > 60:
            raise RuntimeError("no root info")
        time.sleep(0.05)
    return open(path, "rb").read()


def rnd(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.rand(n, device="cuda", generator=g) * 2 - 1).to(dtype)


def scenario_collectives(comm, rank, world):
    for registered in (False, True):
        for dtype in (torch.float32, torch.bfloat16):
            for n in (8, 1000, 65536, 1 << 20, (1 << 22) + 16):
                xs = [rnd(n, dtype, 10 + r) for r in range(world)]   # every rank can build all inputs: the reference is local
                ref = torch.stack([x.double() for x in xs]).sum(0)
                if registered:
                    x = comm.empty((n,), dtype); x.copy_(xs[rank])
                    y = comm.empty((n,), dtype)
                else:
                    x, y = xs[rank].clone(), torch.empty(n, device="cuda", dtype=dtype)
                comm.all_reduce(x, y)
                torch.cuda.synchronize()
                tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
                torch.testing.assert_close(y.double(), ref, rtol=tol, atol=tol * world)
                alg_ar = comm.last_algorithm()
                # all-gather / reduce-scatter
                g = comm.empty((n * world,), dtype) if registered else torch.empty(n * world, device="cuda", dtype=dtype)
                comm.all_gather(x, g)
                torch.cuda.synchronize()
                assert torch.equal(g.view(-1, n)[(rank + 1) % world], xs[(rank + 1) % world])
                big = [rnd(n * world, dtype, 50 + r) for r in range(world)]
                if registered:
                    b = comm.empty((n * world,), dtype); b.copy_(big[rank])
                else:
                    b = big[rank]
                o = torch.empty(n, device="cuda", dtype=dtype)
                comm.reduce_scatter(b, o)
                torch.cuda.synchronize()
                refrs = torch.stack([t.double() for t in big]).sum(0)[rank * n:(rank + 1) * n]
                torch.testing.assert_close(o.double(), refrs, rtol=tol, atol=tol * world)
                if rank == 0:
                    print(f"ok registered={registered} {dtype} n={n} AR={alg_ar} RS={comm.last_algorithm()}", flush=True)
    # broadcast, all-to-all, send/recv ring, barrier
    n = 123457
    b = rnd(n, torch.float32, 7 if rank == 1 % world else 70 + rank)
    comm.broadcast(b, 1 % world)
    torch.cuda.synchronize()
    assert torch.equal(b, rnd(n, torch.float32, 7))
    s = rnd(n * world, torch.float32, 300 + rank)
    r = torch.empty_like(s)
    comm.all_to_all(s, r)
    torch.cuda.synchronize()
    for q in range(world):
        assert torch.equal(r[q * n:(q + 1) * n], rnd(n * world, torch.float32, 300 + q)[rank * n:(rank + 1) * n])
    out = torch.empty(n, device="cuda")
    comm.batch_send_recv([("send", s[:n].contiguous(), (rank + 1) % world), ("recv", out, (rank - 1) % world)])
    torch.cuda.synchronize()
    assert torch.equal(out, rnd(n * world, torch.float32, 300 + (rank - 1) % world)[:n])
    if world >= 2:
        if rank == 0:
            comm.send(s[:1000].contiguous(), 1)
        elif rank == 1:
            got = torch.empty(1000, device="cuda")
            comm.recv(got, 0)
            torch.cuda.synchronize()
            assert torch.equal(got, rnd(n * world, torch.float32, 300)[:1000])
    comm.barrier()
    torch.cuda.synchronize()
    assert comm.async_error() == hb.Result.SUCCESS


def scenario_mc2(comm, rank, world):
    from hccl_b200.ops import mc2

    torch.manual_seed(1234)      # every rank builds all operands: the reference is computed locally in fp32
    # (512, 1280, 512) and (2048, 7168, 256) take narrower column tiles (fewest waves x width): 160 and 224 columns at
    # two ranks; the last shape is the one the benchmarks time (8192 x 3584 x 8192 over all ranks)
    for (m_per, n, k) in ((128, 256, 256), (256, 768, 512), (512, 1024, 1024), (512, 1280, 512), (2048, 7168, 256),
                          (8192 // world, 3584, 8192)):
        shards = [(torch.randn(m_per, k, device="cuda") * 0.5).bfloat16() for _ in range(world)]
        w = (torch.randn(n, k, device="cuda") * 0.1).bfloat16()          # [N, K]
        a = comm.empty((m_per, k), torch.bfloat16)
        a.copy_(shards[rank])
        full = torch.cat(shards)
        ref = full.float() @ w.float().t()
        for rep in range(3):          # pull form: the shard is symmetric memory, the gathered buffer is not
            out, gathered = mc2.all_gather_matmul(comm, a, w)
            torch.cuda.synchronize()
            assert torch.equal(gathered, full), "gathered activations differ"
            err = (out.float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-2, f"AG-matmul err {err}"
        g_sym = comm.empty((m_per * world, k), torch.bfloat16)
        for rep in range(3):          # push form: the gathered buffer is symmetric memory, the shard is a plain tensor;
            # no worker CTAs (the epilogue warps copy) unless HCCL_MC2_AG_WORKERS asks for them
            g_sym.zero_()
            torch.cuda.synchronize()
            out, gathered = mc2.all_gather_matmul(comm, shards[rank], w, gathered=g_sym)
            torch.cuda.synchronize()
            assert torch.equal(gathered, full), "gathered activations differ (push form)"
            err = (out.float() - ref).abs().max().item()
            assert err <= 2e-2 * ref.abs().max().item() + 1e-2, f"AG-matmul (push form) err {err}"
        # matmul -> reduce-scatter: every rank has its own A [M, K] and W [N, K]
        M = m_per * world
        As = [(torch.randn(M, k, device="cuda") * 0.5).bfloat16() for _ in range(world)]
        Ws = [(torch.randn(n, k, device="cuda") * 0.1).bfloat16() for _ in range(world)]
        ref = sum(A.float() @ W.float().t() for A, W in zip(As, Ws))
        for rep in range(3):
            out = mc2.matmul_reduce_scatter(comm, As[rank], Ws[rank])
            torch.cuda.synchronize()
            mine = ref[rank * m_per:(rank + 1) * m_per]
            err = (out.float() - mine).abs().max().item()
            assert err <= 3e-2 * ref.abs().max().item() + 2e-2, f"matmul-RS err {err}"
        # [K, N] weights (the backward layouts)
        Wkn = [W.t().contiguous() for W in Ws]
        out = mc2.matmul_reduce_scatter(comm, As[rank], Wkn[rank], weight_is_kn=True)
        torch.cuda.synchronize()
        err = (out.float() - ref[rank * m_per:(rank + 1) * m_per]).abs().max().item()
        assert err <= 3e-2 * ref.abs().max().item() + 2e-2, f"matmul-RS (KN) err {err}"
        # the backward form of the row-parallel layer: gathered dy times a [K, N] weight
        Wkn0 = Ws[0].t().contiguous()                        # [k, n]: A [M, k] x [k, n]
        g_sym.zero_()
        out, gathered = mc2.all_gather_matmul(comm, shards[rank], Wkn0, weight_is_kn=True, gathered=g_sym)
        torch.cuda.synchronize()
        ref = full.float() @ Wkn0.float()
        err = (out.float() - ref).abs().max().item()
        assert torch.equal(gathered, full) and err <= 2e-2 * ref.abs().max().item() + 1e-2, f"AG-matmul (KN, push) err {err}"
        comm.free(g_sym)
        comm.free(a)
        if rank == 0:
            print(f"mc2 ok m_per={m_per} n={n} k={k}", flush=True)
    # matmul -> all-reduce, decode shapes
    for M in (16, 64, 256):
        k, n = 1024, 2048
        As = [(torch.randn(M, k, device="cuda") * 0.5).bfloat16() for _ in range(world)]
        Ws = [(torch.randn(n, k, device="cuda") * 0.1).bfloat16() for _ in range(world)]
        ref = sum(A.float() @ W.float().t() for A, W in zip(As, Ws))
        for rep in range(4):
            out = mc2.matmul_all_reduce(comm, As[rank], Ws[rank])
            torch.cuda.synchronize()
            err = (out.float() - ref).abs().max().item()
            assert err <= 3e-2 * ref.abs().max().item() + 2e-2, f"matmul-AR err {err} M={M}"
        if rank == 0:
            print(f"mc2 AR ok M={M}", flush=True)
    assert comm.async_error() == hb.Result.SUCCESS


def scenario_graph(comm, rank, world):
    """Collectives captured into a CUDA graph and replayed: the epochs live in device memory, so a replay
    synchronises like a fresh launch."""
    n = 1 << 16
    x = comm.empty((n,), torch.float32)
    y = comm.empty((n,), torch.float32)
    small = torch.ones(64, device="cuda")
    x.fill_(float(rank + 1))
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        comm.all_reduce(x, y)              # warm-up outside capture (first-call checks, plan cache)
        comm.all_reduce(small)
        torch.cuda.synchronize()
        small.fill_(1.0)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            comm.all_reduce(x, y)          # two-shot / one-shot path on symmetric buffers
            comm.all_reduce(small)         # LL path
            comm.barrier()
    want = world * (world + 1) / 2
    acc = 1.0
    for it in range(6):
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        acc *= world
        assert float(y[0]) == want and float(y[-1]) == want, (it, float(y[0]))
        assert float(small[0]) == acc, (it, float(small[0]), acc)
    assert comm.async_error() == hb.Result.SUCCESS
    if rank == 0:
        print("graph replay ok", flush=True)


def scenario_peer_exit(comm, rank, world):
    """A rank leaves between steps; the survivors' next collective ends with an
    error within the wait budget instead of hanging."""
    x = torch.ones(1024, device="cuda")
    comm.all_reduce(x)
    torch.cuda.synchronize()
    assert float(x[0]) == world
    if rank == world - 1:
        torch.cuda.synchronize()
        os._exit(0)            # leaves with nothing in flight
    time.sleep(1.0)
    t0 = time.time()
    failed = False
    try:
        comm.all_reduce(x)
        torch.cuda.synchronize()
        failed = comm.async_error() != hb.Result.SUCCESS
    except hb.HcclError:
        failed = True
    assert failed, "the collective after a peer left must report an error"
    assert time.time() - t0 < 30
    y = torch.ones(4, device="cuda") * 3          # the context is still usable
    assert float(y.sum()) == 12.0
    print(f"rank {rank}: peer exit detected after {time.time() - t0:.2f}s", flush=True)
    os._exit(0)


def scenario_register(comm, rank, world):
    """Buffers the caller allocated itself, registered collectively: operators use them in place on the peers."""
    n = 1 << 20
    g = [torch.Generator(device="cuda").manual_seed(70 + r) for r in range(world)]
    xs = [torch.rand(n, device="cuda", generator=g[r]) for r in range(world)]
    src = torch.empty(n, device="cuda")
    dst = torch.empty(n * world, device="cuda")
    comm.register(src)
    comm.register(dst)
    for rep in range(2):
        src.copy_(xs[rank])
        comm.all_reduce(src, dst[:n])
        torch.cuda.synchronize()
        assert "Nvls" not in comm.last_algorithm(), comm.last_algorithm()      # no multicast alias: peer-to-peer kernels, zero copy
        torch.testing.assert_close(dst[:n], torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)
        comm.all_gather(src, dst)
        torch.cuda.synchronize()
        assert torch.equal(dst, torch.cat(xs))
        per = n // world
        comm.reduce_scatter(src, dst[:per])
        torch.cuda.synchronize()
        torch.testing.assert_close(dst[:per], torch.stack(xs).sum(0)[rank * per:(rank + 1) * per], rtol=1e-5, atol=1e-5)
    comm.deregister(src)
    comm.deregister(dst)
    comm.all_reduce(src, dst[:n])                  # still works, staged again
    torch.cuda.synchronize()
    torch.testing.assert_close(dst[:n], torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)
    assert comm.async_error() == hb.Result.SUCCESS


def scenario_skew(comm, rank, world):
    """Ranks out of step and buffers that differ from rank to rank.
    * runs of small broadcasts while the receivers lag behind the root (the flag-in-data form: a root must not run
      over lines a receiver has not read);
    * in-place AllReduce on symmetric memory at sizes that select the one-shot form;
    * one rank with a 4-byte aligned view, the others with 16-byte aligned tensors;
    * AlltoAllV on ordinary buffers four times the staging window."""
    n = 1024
    busy = torch.empty(1 << 26, device="cuda")
    for rep in range(3):
        bufs = []
        for it in range(6):
            root = (rep + it) % world
            b = rnd(n, torch.float32, 1000 + 10 * rep + it) if rank == root else torch.zeros(n, device="cuda")
            if rank != root:
                for _ in range(3):
                    busy.add_(1.0)                   # the receivers' stream is behind the root's
            comm.broadcast(b, root)
            bufs.append(b)
        torch.cuda.synchronize()
        for it, b in enumerate(bufs):
            assert torch.equal(b, rnd(n, torch.float32, 1000 + 10 * rep + it)), f"broadcast {rep}/{it}"
    assert comm.async_error() == hb.Result.SUCCESS
    for dtype in (torch.float32, torch.bfloat16):
        for m in (8, 3000, 40000, 300000, 1 << 21):
            xs = [rnd(m, dtype, 20 + r) for r in range(world)]
            x = comm.empty((m,), dtype)
            for rep in range(3):
                x.copy_(xs[rank])
                if rank % 2 == 1:
                    busy.add_(1.0)
                comm.all_reduce(x)
                torch.cuda.synchronize()
                tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
                torch.testing.assert_close(x.double(), torch.stack([t.double() for t in xs]).sum(0), rtol=tol, atol=tol * world)
            if rank == 0:
                print(f"in-place symmetric {dtype} n={m}: {comm.last_algorithm()}", flush=True)
            comm.free(x)
    for m in (1000, 100000, 1 << 21):
        xs = [rnd(m + 4, torch.float32, 60 + r) for r in range(world)]
        x = xs[rank][1:1 + m] if rank == 1 else xs[rank][:m]
        y = torch.empty(m + 4, device="cuda")[(1 if rank == 1 else 0):][:m]
        comm.all_reduce(x, y)
        torch.cuda.synchronize()
        want = torch.stack([(t[1:1 + m] if r == 1 else t[:m]).double() for r, t in enumerate(xs)]).sum(0)
        torch.testing.assert_close(y.double(), want, rtol=1e-5, atol=1e-5)
    unit = (64 << 20) // world          # elements of 4 bytes: 4x a pair's window of the 64 MiB slab
    sc = [[unit // 2 + 100 * ((r + 2 * q) % 5) + 3 for q in range(world)] for r in range(world)]
    rc = [sc[q][rank] for q in range(world)]
    sd = [sum(sc[rank][:q]) for q in range(world)]
    rd = [sum(rc[:q]) for q in range(world)]
    src = rnd(sum(sc[rank]), torch.float32, 700 + rank)
    out = torch.zeros(sum(rc), device="cuda")
    comm.all_to_all_v(src, sc[rank], sd, out, rc, rd)
    torch.cuda.synchronize()
    for q in range(world):
        peer = rnd(sum(sc[q]), torch.float32, 700 + q)
        off = sum(sc[q][:rank])
        assert torch.equal(out[rd[q]:rd[q] + rc[q]], peer[off:off + sc[q][rank]]), f"alltoallv block {q}->{rank}"
    assert comm.async_error() == hb.Result.SUCCESS


def scenario_switch_forms(comm, rank, world):
    """AllGather through the switch (symmetric and ordinary outputs), Broadcast as scatter + switch AllGather, and the
    cast + scale reductions over the real transport."""
    import os

    from hccl_b200._lib import lib

    os.environ["HCCL_ALGO"] = "allgather=level0:nvls"
    lib.HcclReloadEnvConfig()
    for n in (4096, 300000, 1 << 22):
        xs = [rnd(n, torch.float32, 40 + r) for r in range(world)]
        for sym in (False, True):
            out = comm.empty((n * world,), torch.float32) if sym else torch.empty(n * world, device="cuda")
            for rep in range(2):
                out.zero_()
                comm.all_gather(xs[rank], out)
                torch.cuda.synchronize()
                assert torch.equal(out, torch.cat(xs)), f"switch allgather n={n} sym={sym}"
            if rank == 0:
                print(f"allgather n={n} sym={sym}: {comm.last_algorithm()}", flush=True)
            if sym:
                comm.free(out)
    os.environ.pop("HCCL_ALGO")
    lib.HcclReloadEnvConfig()
    for n in (1 << 19, (1 << 22) + 4):
        for root in (0, world - 1):
            for sym in (False, True):
                b = comm.empty((n,), torch.float32) if sym else torch.empty(n, device="cuda")
                b.copy_(rnd(n, torch.float32, 5) if rank == root else torch.zeros(n, device="cuda"))
                comm.broadcast(b, root)
                torch.cuda.synchronize()
                assert torch.equal(b, rnd(n, torch.float32, 5)), f"broadcast n={n} root={root} sym={sym}"
                if rank == 0:
                    print(f"broadcast n={n} root={root} sym={sym}: {comm.last_algorithm()}", flush=True)
                if sym:
                    comm.free(b)
    for n in (1000, 1 << 21):
        xs = [rnd(n, torch.float32, 70 + r) for r in range(world)]
        y = torch.empty(n, device="cuda", dtype=torch.bfloat16)
        comm.all_reduce_ex(xs[rank], y, scale=1.0 / world)
        torch.cuda.synchronize()
        torch.testing.assert_close(y.double(), torch.stack([t.double() for t in xs]).mean(0), rtol=1e-2, atol=1e-2)
        g = comm.empty((n,), torch.float32)
        g.copy_(xs[rank])
        comm.all_reduce_ex(g, scale=1.0 / world)
        torch.cuda.synchronize()
        torch.testing.assert_close(g.double(), torch.stack([t.double() for t in xs]).mean(0), rtol=1e-6, atol=1e-6)
        comm.free(g)
    s = rnd(300000 * world, torch.float32, 300 + rank)
    r = torch.empty_like(s)
    for rep in range(3):
        comm.all_to_all(s, r)
        torch.cuda.synchronize()
        for q in range(world):
            assert torch.equal(r[q * 300000:(q + 1) * 300000], rnd(300000 * world, torch.float32, 300 + q)[rank * 300000:(rank + 1) * 300000])
    if rank == 0:
        print(f"alltoall 300000 floats per pair: {comm.last_algorithm()}", flush=True)
    assert comm.async_error() == hb.Result.SUCCESS


def scenario_model(rank, world, path):
    """Two-layer TP+SP decoder stack: loss and gradients of the NCCL + cuBLAS arm against the same model in one piece,
    and of the fused-kernel arm against the NCCL + cuBLAS arm, for both AllGather->Matmul forms; two steps each
    (persistent symmetric buffers are reused)."""
    import torch.distributed as dist

    from hccl_b200.models import LlamaConfig, LlamaStack
    from hccl_b200.parallel import TPContext

    store = dist.FileStore(path + ".store", world)
    dist.init_process_group("nccl", rank=rank, world_size=world, store=store, device_id=torch.device("cuda", torch.cuda.current_device()))
    comm = Communicator.from_torch_distributed(config=hb.make_config(buffer_mib=64))
    cfg = LlamaConfig.tiny(2)
    seq = 128 * world
    tokens = torch.randint(0, cfg.vocab, (seq,), generator=torch.Generator().manual_seed(5), dtype=torch.int64).cuda()

    # the same model in one piece (this library's matmul kernels on one GPU), built from one seed on every rank
    one_ctx = TPContext(comm=None, impl="hccl")
    torch.manual_seed(77)
    one = LlamaStack(cfg, one_ctx)
    with torch.no_grad():
        for p_ in one.replicated_parameters():
            p_.add_(0.1 * torch.randn_like(p_))
    one_loss = one.loss(tokens)
    one_loss.backward()
    holder_src = LlamaStack(cfg, one_ctx)
    with torch.no_grad():
        for (n_, p_), (_, q_) in zip(holder_src.named_parameters(), one.named_parameters()):
            p_.copy_(q_.grad)

    def run(impl, form):
        os.environ["HCCL_TP_AG_FORM"] = form
        ctx = TPContext(comm=comm if impl == "hccl" else None, group=None, impl=impl)
        model = LlamaStack(cfg, ctx)
        model.load_full(one)
        out = []
        for _ in range(2):
            model.zero_grad(set_to_none=True)
            loss = model.loss(tokens)
            loss.backward()
            model.sync_replicated_grads()
            total = loss.detach().clone()
            dist.all_reduce(total)
            torch.cuda.synchronize()
            out.append((total.item(), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None}))
        want = LlamaStack(cfg, ctx)
        want.load_full(holder_src)                      # this rank's slices of the one-piece gradients
        ctx.release()
        return out, {n: p.detach().float() for n, p in want.named_parameters()}

    ref, want = run("nccl", "pull")
    # the framework arm against the model in one piece: loss and every gradient (sharded and replicated)
    assert abs(ref[0][0] - one_loss.item()) <= 2e-2 * abs(one_loss.item()) + 1e-4, f"loss {ref[0][0]} vs one-piece {one_loss.item()}"
    for name, g in ref[0][1].items():
        denom = want[name].abs().max().item() + 1e-8
        err = (g - want[name]).abs().max().item() / denom
        assert err <= 8e-2, f"grad {name} differs from the one-piece model by {err:.3f} of its max"
    for form in ("push", "pull"):
        got, _ = run("hccl", form)
        for step, ((l0, g0), (l1, g1)) in enumerate(zip(ref, got)):
            assert abs(l0 - l1) <= 2e-2 * abs(l0) + 1e-4, f"{form} step {step}: loss {l1} vs {l0}"
            for name in g0:
                denom = g0[name].abs().max().item() + 1e-8
                err = (g0[name] - g1[name]).abs().max().item() / denom
                assert err <= 6e-2, f"{form} step {step}: grad {name} differs by {err:.3f} of its max"
    comm.destroy()
    dist.destroy_process_group()
    print(f"rank {rank} model ok", flush=True)


def scenario_torch_backend(rank, world, path):
    """Unmodified torch.distributed calls on the "hccl" backend, compared with local references."""
    import torch.distributed as dist

    import hccl_b200.torch_backend  # noqa: F401  (registers the backend)

    store = dist.FileStore(path + ".store", world)
    dist.init_process_group("hccl", rank=rank, world_size=world, store=store)
    assert dist.get_backend() == "hccl"
    dev = torch.device("cuda", torch.cuda.current_device())
    g = [torch.Generator(device="cuda").manual_seed(50 + r) for r in range(world)]
    xs = [torch.rand(5000, device="cuda", generator=g[r]) for r in range(world)]       # every rank can rebuild all inputs
    t = xs[rank].clone()
    dist.all_reduce(t)
    torch.testing.assert_close(t, torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)
    t = xs[rank].clone()
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert torch.equal(t, torch.stack(xs).max(0).values)
    b = xs[rank].clone()
    dist.broadcast(b, src=world - 1)
    assert torch.equal(b, xs[world - 1])
    out = torch.empty(world * 5000, device="cuda")
    dist.all_gather_into_tensor(out, xs[rank])
    assert torch.equal(out, torch.cat(xs))
    outs = [torch.empty(5000, device="cuda") for _ in range(world)]
    dist.all_gather(outs, xs[rank])
    assert all(torch.equal(o, x) for o, x in zip(outs, xs))
    n = 5000 // world * world
    rs = torch.empty(n // world, device="cuda")
    dist.reduce_scatter_tensor(rs, xs[rank][:n].contiguous())
    want = torch.stack([x[:n] for x in xs]).sum(0)[rank * (n // world):(rank + 1) * (n // world)]
    torch.testing.assert_close(rs, want, rtol=1e-5, atol=1e-5)
    a2a = torch.empty(n, device="cuda")
    dist.all_to_all_single(a2a, xs[rank][:n].contiguous())
    per = n // world
    assert torch.equal(a2a, torch.cat([xs[q][rank * per:(rank + 1) * per] for q in range(world)]))
    r = xs[rank].clone()
    dist.reduce(r, dst=0)
    if rank == 0:
        torch.testing.assert_close(r, torch.stack(xs).sum(0), rtol=1e-5, atol=1e-5)
    if rank == 0:
        dist.send(xs[0], dst=1)
    elif rank == 1:
        got = torch.empty(5000, device="cuda")
        dist.recv(got, src=0)
        assert torch.equal(got, xs[0])
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()
    print(f"rank {rank} torch backend ok on {dev}", flush=True)


def main():
    rank, world, path, scenario = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4]
    torch.cuda.set_device(rank % torch.cuda.device_count())
    if scenario in ("torch_backend", "model"):
        {"torch_backend": scenario_torch_backend, "model": scenario_model}[scenario](rank, world, path)
        print(f"rank {rank} done", flush=True)
        return
    info = rendezvous(rank, path)
    timeout_ms = 3000 if scenario == "peer_exit" else 0
    comm = Communicator.from_root_info(info, rank, world, hb.make_config(buffer_mib=64, exec_timeout_ms=timeout_ms))
    {"collectives": scenario_collectives, "skew": scenario_skew, "switch_forms": scenario_switch_forms, "peer_exit": scenario_peer_exit, "mc2": scenario_mc2, "graph": scenario_graph,
     "register": scenario_register}[scenario](comm, rank, world)
    comm.destroy()
    print(f"rank {rank} done", flush=True)


if __name__ == "__main__":
    main()
