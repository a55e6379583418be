"""Data-parallel training of a small MLP on this library's operators: gradients are packed into flat buckets and
all-reduced on a side stream while backward is still running (`GradientBucketer`), the update runs as one kernel
launch (`FusedAdamW`).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29502 \\
        examples/03_pytorch/data_parallel_training.py

Every rank draws its own batch; after each step all replicas hold the same parameters, which the script checks.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.ops.functional as hdist  # noqa: E402
from hccl_b200.ops import FusedAdamW  # noqa: E402
from hccl_b200.parallel import GradientBucketer  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo", rank=rank, world_size=world)   # only hands out the root info
comm = hdist.init_process_group()

torch.manual_seed(0)                                            # the same initial weights everywhere
model = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.GELU(), torch.nn.Linear(4096, 4096), torch.nn.GELU(),
                            torch.nn.Linear(4096, 1024)).cuda().bfloat16()
opt = FusedAdamW(model.parameters(), lr=1e-3)
sync = GradientBucketer(model.parameters(), comm, bucket_mib=8, overlap=True)
gen = torch.Generator(device="cuda").manual_seed(100 + rank)    # a different batch on every rank

for step in range(10):
    x = torch.randn(256, 1024, device="cuda", generator=gen).bfloat16()
    model.zero_grad(set_to_none=True)
    loss = model(x).float().pow(2).mean()
    loss.backward()                                             # buckets are all-reduced as they fill up
    sync.finish()                                               # wait, average, write back
    opt.step()
    if rank == 0 and step % 3 == 0:
        print(f"step {step}: loss {loss.item():.5f}, {len(sync.buckets)} buckets")

# all replicas agree bit for bit: same start, same averaged gradients, same update
probe = torch.cat([p.detach().float().reshape(-1)[:16] for p in model.parameters()])
low, high = probe.clone(), probe.clone()
hdist.all_reduce(low, op="min")
hdist.all_reduce(high, op="max")
torch.cuda.synchronize()
print(f"rank {rank}: replicas identical = {bool(torch.equal(low, high))}")
hdist.destroy_process_group()
dist.destroy_process_group()
