"""Expert-parallel MoE forward on AlltoAll / AlltoAllV (`moe_forward`): every GPU hosts E / P experts, tokens go to
the ranks of their top-k experts and the weighted outputs come back.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29505 \\
        examples/03_pytorch/expert_parallel_moe.py

For the fused path (token permutation and fp8 block quantisation inside the transfer, gate-weighted sum inside the
pull) see `hccl_b200.ops.moe.MoeDispatcher` and `bench/moe_bench.py`.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.ops.functional as hdist  # noqa: E402
from hccl_b200.parallel import moe_forward  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo", rank=rank, world_size=world)   # only hands out the root info
comm = hdist.init_process_group()

tokens, hidden, topk, e_local = 2048, 1024, 2, 4
n_experts = e_local * world
torch.manual_seed(1000 + rank)
weights = [torch.randn(hidden, hidden, device="cuda", dtype=torch.bfloat16) / hidden ** 0.5 for _ in range(e_local)]
experts = [(lambda w: (lambda rows: torch.nn.functional.gelu(rows @ w)))(w) for w in weights]
x = torch.randn(tokens, hidden, device="cuda", dtype=torch.bfloat16)
router = torch.randn(tokens, n_experts, device="cuda")
gate, idx = torch.topk(torch.softmax(router, dim=-1), topk, dim=-1)
gate = gate / gate.sum(-1, keepdim=True)

out = moe_forward(x, idx.int(), gate, experts, comm, n_experts)
torch.cuda.synchronize()
print(f"rank {rank}: output {tuple(out.shape)} {out.dtype}, mean |y| = {out.float().abs().mean().item():.4f}")
hdist.destroy_process_group()
dist.destroy_process_group()
