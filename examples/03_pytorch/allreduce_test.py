"""PyTorch usage (the counterpart of HCCL's examples/03_ai_framework/01_pytorch/hccl_pytorch_allreduce_test.py).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29501 \
        examples/03_pytorch/allreduce_test.py
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.ops.functional as hdist  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo", rank=rank, world_size=world)   # any backend: only used to hand out the root info
comm = hdist.init_process_group()
x = torch.full((1 << 20,), float(rank + 1), device="cuda")
hdist.all_reduce(x)
torch.cuda.synchronize()
print(f"rank {rank}: {x[0].item()} (expected {world * (world + 1) / 2}) via {comm.last_algorithm()}")
# symmetric (zero-copy) tensors: peers read them in place
y = comm.empty((1 << 20,), torch.bfloat16)
y.fill_(1.0)
hdist.all_reduce(y)
torch.cuda.synchronize()
print(f"rank {rank}: symmetric {y[0].item()} via {comm.last_algorithm()}")
hdist.destroy_process_group()
dist.destroy_process_group()
