"""Single-pass element-wise kernels of the decoder stack against the PyTorch expressions they replace (one GPU).

    python bench/fused_ops_bench.py [--rows 4096] [--hidden 8192] [--ffn 28672] [--iters 20] [--only NAME] [--adam-params N]

Shapes of the Llama-3-70B block at sequence 4096: residual add + RMSNorm on [rows, hidden], SwiGLU on
[rows, 2 * ffn], rotary embedding on 64 heads of 128.  Forward + backward per op, CUDA events, 5 warm-up + `iters`
timed calls; a 256 MiB buffer is rewritten between calls so that every call starts with a cold L2.  Prints one JSON row
per op with the algorithmic bytes (each tensor read or written once), the achieved GB/s and the same for the PyTorch
expression.  `--only NAME` runs one op a few times without the comparison (for profiling one kernel in isolation).
The `adamw` row is the optimizer update over 24 bf16 tensors of `--adam-params` elements in total (bf16 moments, 14
bytes per parameter) against torch.optim.AdamW(fused=True).
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from hccl_b200.ops import fused  # noqa: E402


def timed(fn, iters, flush):
    for _ in range(5):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=28672)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--only", default="")
    ap.add_argument("--adam-params", type=int, default=1 << 29, help="parameters of the adamw row (default 512 Mi: 7.5 GB moved per call)")
    args = ap.parse_args()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    R, H, Fd, NH, D = args.rows, args.hidden, args.ffn, args.heads, args.head_dim
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def rnd(*shape):
        return torch.randn(*shape, device="cuda", generator=g).bfloat16()

    x, delta, w = rnd(R, H).requires_grad_(), rnd(R, H).requires_grad_(), (1 + 0.1 * rnd(H).float()).bfloat16().requires_grad_()
    up_h, up_x = rnd(R, H), rnd(R, H)
    gu, up_o = rnd(R, 2 * Fd).requires_grad_(), rnd(R, Fd)
    q, up_q = rnd(R, NH, D).requires_grad_(), rnd(R, NH, D)
    ang = torch.rand(R, D // 2, device="cuda", generator=g) * 6.28
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()

    def norm(use):
        def f():
            xo, h = fused.add_rms_norm(x, delta, w, 1e-5, use_kernels=use)
            torch.autograd.backward([xo, h], [up_x, up_h])
            x.grad = delta.grad = w.grad = None
        return f

    def swi(use):
        def f():
            o = fused.swiglu(gu, use_kernels=use)
            o.backward(up_o)
            gu.grad = None
        return f

    def rope(use):
        def f():
            o = fused.rope(q, cos, sin, use_kernels=use)
            o.backward(up_q)
            q.grad = None
        return f

    # algorithmic bytes, forward + backward, every tensor once (bf16 = 2 bytes)
    cases = {
        "add_rms_norm": (norm, (4 * R * H + 4 * R * H) * 2),   # fwd: x, delta in; x_out, h out / bwd: dh, dx_out, x_out in; dx out (the same dx serves x and delta)
        "swiglu": (swi, (2 * R * Fd + R * Fd) * 2 + (2 * R * Fd + R * Fd + 2 * R * Fd) * 2),
        "rope": (rope, 2 * R * NH * D * 2 * 2),
    }
    # optimizer: the same update with this library's kernel and with PyTorch's fused multi-tensor AdamW
    from hccl_b200.ops import FusedAdamW
    per = max(8, args.adam_params // 24)
    adam_state = {}

    def adam(use):
        if use not in adam_state:
            ps = [torch.nn.Parameter(rnd(per)) for _ in range(24)]
            for p_ in ps:
                p_.grad = rnd(per)
            opt = FusedAdamW(ps, lr=1e-4) if use else torch.optim.AdamW(ps, lr=1e-4, fused=True)
            adam_state[use] = (ps, opt)
        return adam_state[use][1].step

    if not args.only or args.only == "adamw":
        cases["adamw"] = (adam, 24 * per * 14)
    for name, (mk, nbytes) in cases.items():
        if args.only and args.only != name:
            continue
        if args.only:
            for _ in range(3):
                mk(True)()
            torch.cuda.synchronize()
            continue
        t_k = timed(mk(True), args.iters, flush)
        t_t = timed(mk(False), args.iters, flush)
        print(json.dumps({"op": name, "rows": R, "kernels_ms": t_k, "torch_ms": t_t, "speedup": t_t / t_k, "algorithmic_MB": nbytes / 1e6,
                          "kernels_GBs": nbytes / t_k / 1e6, "torch_GBs": nbytes / t_t / 1e6}), flush=True)


if __name__ == "__main__":
    main()
