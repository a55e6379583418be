"""The tensor + sequence parallel decoder stack against the same model in one piece.

Ranks are CPU processes on the gloo backend (the framework arm of the layers: torch.distributed collectives and
torch.matmul), fp32, so the comparison is tight.  Every rank cuts its shards out of the one-piece model built from the
same seed; the summed per-rank losses, every sharded gradient (compared with the matching slice of the one-piece
gradient) and the gradients of the replicated RMSNorm weights after ``sync_replicated_grads`` have to agree.  The
fused-kernel arm is compared with this arm on GPUs (``scenario_model``), so the two together tie it to the one-piece
model.
"""
import os
import sys
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _build(cfg, ctx, seed):
    from hccl_b200.models import LlamaStack

    torch.manual_seed(seed)
    model = LlamaStack(cfg, ctx)
    # norm weights away from 1 so that their gradients and their use are both exercised
    with torch.no_grad():
        for p in model.replicated_parameters():
            p.add_(0.1 * torch.randn_like(p))
    return model


def _grad_slices(full_grad, model, full_model):
    """This rank's slices of the one-piece gradients, cut exactly as the parameters are: load_full applied to a copy of
    the one-piece model whose parameters hold its gradients."""
    grads = type(full_model)(full_model.cfg, full_model.ctx)
    with torch.no_grad():
        for n, p in grads.named_parameters():
            p.copy_(full_grad[n])
    holder = type(model)(model.cfg, model.ctx)
    holder.load_full(grads)
    return {n: p.detach() for n, p in holder.named_parameters()}


def _worker(rank, world, store_path, out_path):
    sys.path.insert(0, ROOT)
    from hccl_b200.models import LlamaConfig
    from hccl_b200.parallel import TPContext

    store = dist.FileStore(store_path, world)
    dist.init_process_group("gloo", rank=rank, world_size=world, store=store)
    torch.set_num_threads(2)
    cfg = LlamaConfig(hidden=64, n_heads=8, n_kv_heads=4, head_dim=8, ffn=128, n_layers=2, vocab=96, init_std=0.2)
    seq = 16 * world
    tokens = torch.randint(0, cfg.vocab, (seq,), generator=torch.Generator().manual_seed(3))

    full_ctx = TPContext(impl="nccl", device="cpu", dtype=torch.float32, group=dist.new_group([rank]))
    assert full_ctx.world == 1
    full = _build(cfg, full_ctx, seed=11)
    full_loss = full.loss(tokens)
    full_loss.backward()
    full_grad = {n: p.grad.clone() for n, p in full.named_parameters()}

    ctx = TPContext(impl="nccl", device="cpu", dtype=torch.float32)
    assert ctx.world == world and ctx.rank == rank
    model = _build(cfg, ctx, seed=100 + rank)          # different values, then overwritten by the slices
    model.load_full(full)
    for step in range(2):
        model.zero_grad(set_to_none=True)
        loss = model.loss(tokens)
        loss.backward()
        model.sync_replicated_grads()
    total = loss.detach().clone()
    dist.all_reduce(total)
    torch.testing.assert_close(total, full_loss.detach(), rtol=1e-5, atol=1e-7)
    worst = 0.0
    slices = _grad_slices(full_grad, model, full)
    for name, p in model.named_parameters():
        want = slices[name]
        assert p.grad is not None, name
        err = (p.grad - want).abs().max().item() / (want.abs().max().item() + 1e-12)
        worst = max(worst, err)
        assert err < 2e-4, f"rank {rank}: gradient of {name} differs from the one-piece model by {err:.2e} of its max"
    # without the sum over the group the replicated gradients are wrong: the check above is not vacuous
    model.zero_grad(set_to_none=True)
    model.loss(tokens).backward()
    p0 = model.replicated_parameters()[0]
    name0 = [n for n, p in model.named_parameters() if p is p0][0]
    assert (p0.grad - full_grad[name0]).abs().max().item() > 1e-3 * full_grad[name0].abs().max().item()
    with open(f"{out_path}.{rank}", "w") as f:
        f.write(f"ok {worst:.3e}")
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tp_sp_stack_matches_the_one_piece_model(world):
    with tempfile.TemporaryDirectory() as d:
        store, out = os.path.join(d, "store"), os.path.join(d, "out")
        mp.spawn(_worker, args=(world, store, out), nprocs=world, join=True)
        for r in range(world):
            assert open(f"{out}.{r}").read().startswith("ok")
