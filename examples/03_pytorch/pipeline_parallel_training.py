"""Pipeline-parallel training on BatchSendRecv: every GPU holds one stage of an MLP; micro-batches flow forward through
the stages and their gradients flow back (`gpipe_step`), then every stage updates its own parameters (`FusedAdamW`).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29504 \\
        examples/03_pytorch/pipeline_parallel_training.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.ops.functional as hdist  # noqa: E402
from hccl_b200.ops import FusedAdamW  # noqa: E402
from hccl_b200.parallel import gpipe_step  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo", rank=rank, world_size=world)   # only hands out the root info
comm = hdist.init_process_group()

width, batch, n_micro = 2048, 64, 8
torch.manual_seed(rank)
stage = torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.GELU(), torch.nn.Linear(width, width)).cuda().bfloat16()
opt = FusedAdamW(stage.parameters(), lr=1e-4)
gen = torch.Generator(device="cuda").manual_seed(1)

for step in range(5):
    inputs = [torch.randn(batch, width, device="cuda", generator=gen).bfloat16() for _ in range(n_micro)] if rank == 0 else None
    opt.zero_grad(set_to_none=True)
    loss = gpipe_step(stage, comm, n_micro, (batch, width), torch.bfloat16, "cuda", inputs=inputs,
                      loss_fn=(lambda y, m: y.float().pow(2).mean()) if rank == world - 1 else None)
    opt.step()
    if rank == world - 1:
        print(f"step {step}: loss {loss.item():.5f}")
torch.cuda.synchronize()
hdist.destroy_process_group()
dist.destroy_process_group()
