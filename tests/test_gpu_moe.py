"""MoE dispatch (fp8 1x128 block-scaled) and combine (gate-weighted sum) with ranks emulated on one GPU, against a
plain PyTorch fp32 reference of the same routing."""
import pytest
import torch

pytestmark = pytest.mark.gpu

import hccl_b200 as hb
from hccl_b200 import Communicator
from hccl_b200.ops.moe import MoeDispatcher, dequantize


@pytest.mark.parametrize("p,tokens,hidden,experts,topk", [(2, 64, 256, 8, 2), (4, 200, 1024, 32, 4), (8, 128, 7168, 256, 8)])
def test_dispatch_combine_emulated(p, tokens, hidden, experts, topk):
    torch.cuda.set_device(0)
    comms = Communicator.emulated(p, hb.make_config(buffer_mib=8))
    per = experts // p
    disp = [MoeDispatcher(c, tokens, hidden, topk, experts) for c in comms]      # rank by rank: symmetric allocations pair up
    xs, idxs, ws = [], [], []
    for r in range(p):
        g = torch.Generator(device="cuda").manual_seed(10 + r)
        xs.append(torch.randn(tokens, hidden, device="cuda", generator=g).bfloat16())
        logits = torch.randn(tokens, experts, device="cuda", generator=g)
        w, i = torch.topk(torch.softmax(logits, -1), topk, dim=-1)
        idxs.append(i.int().contiguous())
        ws.append((w / w.sum(-1, keepdim=True)).float().contiguous())
    res = [d.dispatch(x, i) for d, x, i in zip(disp, xs, idxs)]
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    for r in range(p):
        off = res[r].offsets.cpu().tolist()
        # expected number of rows per local expert
        for le in range(per):
            want = sum(int((idxs[s] == r * per + le).sum()) for s in range(p))
            assert off[le + 1] - off[le] == want
        n = off[-1]
        deq = dequantize(res[r].x_fp8[:n], res[r].scales[:n])
        src = res[r].src_info[:n].cpu()
        srank, pair = (src >> 32).tolist(), (src & 0xFFFFFFFF).tolist()
        for row in range(0, n, max(1, n // 50)):           # sample rows
            t, k = pair[row] // topk, pair[row] % topk
            e = int(idxs[srank[row]][t, k])
            assert e // per == r and off[e % per] <= row < off[e % per + 1]
            ref = xs[srank[row]][t].float()
            assert (deq[row] - ref).abs().max() <= 0.07 * ref.abs().max() + 1e-3     # e4m3: 3 mantissa bits
        # rows of one expert are ordered by source rank
        for le in range(per):
            seg = srank[off[le]:off[le + 1]]
            assert seg == sorted(seg)
    # "experts": expert e multiplies by 1 + (e % 7) / 4, a different factor per expert of a token, so that the combine
    # result depends on WHICH gate weight meets which expert output (a constant factor would hide a wrong pairing)
    def factor(e):
        return 1.0 + (e % 7) / 4.0

    for r in range(p):
        off = res[r].offsets.cpu().tolist()
        n = off[-1]
        deq = dequantize(res[r].x_fp8[:n], res[r].scales[:n])
        for le in range(per):
            deq[off[le]:off[le + 1]] *= factor(r * per + le)
        disp[r].y[:n] = deq.bfloat16()
    outs = [d.combine(w) for d, w in zip(disp, ws)]
    torch.cuda.synchronize()
    for r in range(p):
        f = torch.tensor([[factor(int(e)) if e >= 0 else 0.0 for e in row] for row in idxs[r].cpu().tolist()], device="cuda")
        ref = xs[r].float() * (ws[r].float() * f).sum(1, keepdim=True)
        err = (outs[r].float() - ref).abs().max().item()
        assert err <= 0.08 * ref.abs().max().item() + 1e-2, err
        # the check can tell a wrong pairing: the same sum with the weights of each token rotated by one is far off
        if topk > 1:
            wrong = xs[r].float() * (ws[r].float().roll(1, dims=1) * f).sum(1, keepdim=True)
            assert (wrong - ref).abs().max().item() > 0.1 * ref.abs().max().item()
    # a second round reuses all buffers
    res = [d.dispatch(x, i) for d, x, i in zip(disp, xs, idxs)]
    torch.cuda.synchronize()
    assert comms[0].async_error() == hb.Result.SUCCESS
    for c in comms:
        c.destroy()


@pytest.mark.parametrize("tokens,topk,experts", [(1, 1, 4), (777, 8, 256), (8192, 8, 256), (100000, 2, 4096)])
def test_expert_offsets(tokens, topk, experts):
    from hccl_b200.ops.moe import expert_offsets

    g = torch.Generator(device="cuda").manual_seed(tokens)
    idx = torch.randint(-1, experts, (tokens, topk), device="cuda", generator=g, dtype=torch.int32)
    for _ in range(3):          # repeated calls: the scratch must be clean again after each
        off = expert_offsets(idx, experts)
        torch.cuda.synchronize()
        valid = idx[idx >= 0].long()
        ref = torch.zeros(experts + 1, dtype=torch.int64, device="cuda")
        ref[1:] = torch.bincount(valid, minlength=experts).cumsum(0)
        assert torch.equal(off.long(), ref)
