"""FusedAdamW: the single-launch AdamW kernel against a plain PyTorch fp32 AdamW of the same update."""
import pytest
import torch

from hccl_b200.ops import FusedAdamW
from hccl_b200.ops.optim import adamw_reference_


def _fp32_reference(params0, grads_per_step, lr, betas, eps, wd, round_to):
    """torch.optim.AdamW in fp32 on copies of the parameters; after every step parameters and moments are rounded to the
    storage dtype, which is what a kernel that stores bf16 does."""
    ps = [p.detach().float().clone() for p in params0]
    ms = [torch.zeros_like(p) for p in ps]
    vs = [torch.zeros_like(p) for p in ps]
    for t, grads in enumerate(grads_per_step, 1):
        for p, g, m, v in zip(ps, grads, ms, vs):
            adamw_reference_(p, g.float(), m, v, t, lr, betas[0], betas[1], eps, wd)
            for x in (p, m, v):
                x.copy_(x.to(round_to).float())
    return ps, ms, vs


def test_cpu_path_matches_torch_adamw():
    torch.manual_seed(0)
    ps = [torch.nn.Parameter(torch.randn(37, 5)), torch.nn.Parameter(torch.randn(11))]
    qs = [torch.nn.Parameter(p.detach().clone()) for p in ps]
    a = FusedAdamW(ps, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    b = torch.optim.AdamW(qs, lr=3e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(4):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        a.step()
        b.step()
    for p, q in zip(ps, qs):
        torch.testing.assert_close(p, q, rtol=1e-5, atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("pdt,sdt", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32), (torch.bfloat16, torch.float32)])
def test_kernel_matches_fp32_reference(pdt, sdt):
    torch.manual_seed(1)
    dev = "cuda"
    shapes = [(1024, 1024), (8192,), (333, 77), (1,), (4099,), (256, 8200)]        # vector bodies, ragged tails, a single element
    params = [torch.nn.Parameter((torch.randn(s, device=dev) * 0.05).to(pdt)) for s in shapes]
    lr, betas, eps, wd = 1e-2, (0.9, 0.95), 1e-8, 0.1
    opt = FusedAdamW(params, lr=lr, betas=betas, eps=eps, weight_decay=wd, state_dtype=sdt)
    p0 = [p.detach().clone() for p in params]
    steps = [[(torch.randn(s, device=dev) * 0.1).to(pdt) for s in shapes] for _ in range(3)]
    for grads in steps:
        for p, g in zip(params, grads):
            p.grad = g.clone()
        opt.step()
    torch.cuda.synchronize()
    rp, rm, rv = _fp32_reference(p0, steps, lr, betas, eps, wd, pdt if sdt == pdt else torch.float32)
    if sdt != pdt:      # bf16 parameters, fp32 moments: only the parameters are rounded
        rp, rm, rv = [], [], []
        ps = [p.float().clone() for p in p0]
        ms = [torch.zeros_like(p) for p in ps]
        vs = [torch.zeros_like(p) for p in ps]
        for t, grads in enumerate(steps, 1):
            for p, g, m, v in zip(ps, grads, ms, vs):
                adamw_reference_(p, g.float(), m, v, t, lr, betas[0], betas[1], eps, wd)
                p.copy_(p.to(pdt).float())
        rp, rm, rv = ps, ms, vs
    tol = dict(rtol=2e-2, atol=2e-3) if pdt == torch.bfloat16 else dict(rtol=1e-5, atol=1e-6)
    for p, r in zip(params, rp):
        torch.testing.assert_close(p.detach().float(), r, **tol)
    # bf16 moments: a one-ulp difference in a stored moment (fused multiply-add against separate rounding) is carried
    # into the next step with weight beta, also where the new value cancels to almost nothing; one ulp is 2.4e-4 at
    # |m| <= 0.06 and 7.6e-6 at v <= 2e-3
    mtol = dict(rtol=2e-2, atol=5e-4) if sdt == torch.bfloat16 else dict(rtol=1e-5, atol=1e-7)
    vtol = dict(rtol=2e-2, atol=2e-5) if sdt == torch.bfloat16 else dict(rtol=1e-5, atol=1e-9)
    for p, m, v in zip(params, rm, rv):
        torch.testing.assert_close(opt.state[p]["exp_avg"].float(), m, **mtol)
        torch.testing.assert_close(opt.state[p]["exp_avg_sq"].float(), v, **vtol)
    assert opt.launches == 3 * 2        # per step: the step-counter kernel and one update kernel for all six tensors


@pytest.mark.gpu
def test_more_than_one_batch_of_tensors_and_graph_replay():
    torch.manual_seed(2)
    params = [torch.nn.Parameter(torch.randn(100 + i, device="cuda", dtype=torch.bfloat16)) for i in range(170)]      # three launches of <= 80
    refs = [p.detach().float().clone() for p in params]
    opt = FusedAdamW(params, lr=1e-2, weight_decay=0.0)
    grads = [torch.randn_like(p) for p in params]
    for p, g in zip(params, grads):
        p.grad = g
    opt.step()                                            # eager step 1
    g_ = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g_):
        opt.step()                                        # captured: step 2
    g_.replay()                                           # step 3 (capture itself does not run the kernels)
    g_.replay()
    torch.cuda.synchronize()
    ms = [torch.zeros_like(r) for r in refs]
    vs = [torch.zeros_like(r) for r in refs]
    for t in (1, 2, 3):
        for r, g, m, v in zip(refs, grads, ms, vs):
            adamw_reference_(r, g.float(), m, v, t, 1e-2, 0.9, 0.999, 1e-8, 0.0)
            for x in (r, m, v):
                x.copy_(x.bfloat16().float())
    for p, r in zip(params, refs):
        torch.testing.assert_close(p.detach().float(), r, rtol=3e-2, atol=3e-3)
    assert float(opt.param_groups[0]["step_state"][(torch.bfloat16, torch.bfloat16, params[0].device)][0]) == 3.0
