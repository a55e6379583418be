"""Attention over a sequence that is sharded across GPUs, two ways, on this library's operators:
Ulysses (AlltoAll swaps the sequence shard for a head shard) and ring attention (keys and values travel around the
ring with BatchSendRecv while every rank folds one block per step into its running softmax).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29503 \\
        examples/03_pytorch/context_parallel_attention.py

Every rank holds S / P tokens of a causal sequence; the result is checked against plain attention over the whole
sequence, which rank 0 computes from the gathered inputs.
"""
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.ops.functional as hdist  # noqa: E402
from hccl_b200.parallel import ring_attention, ulysses_attention  # noqa: E402

rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
dist.init_process_group("gloo", rank=rank, world_size=world)   # only hands out the root info
comm = hdist.init_process_group()

s, H, D = 1024, 8 * world, 128                                  # tokens per rank, heads, head size
gen = torch.Generator(device="cuda").manual_seed(7 + rank)
q, k, v = (torch.randn(s, H, D, device="cuda", generator=gen).bfloat16() for _ in range(3))

out_u = ulysses_attention(q, k, v, comm, causal=True)
out_r = ring_attention(q, k, v, comm, causal=True)

# the whole sequence on every rank, for the check
full = [torch.empty(world * s, H, D, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
for dst, src in zip(full, (q, k, v)):
    comm.all_gather(src.contiguous(), dst)
Q, K, V = (t.transpose(0, 1).float() for t in full)
want = F.scaled_dot_product_attention(Q, K, V, is_causal=True).transpose(0, 1)[rank * s:(rank + 1) * s]
torch.cuda.synchronize()
err_u = (out_u.float() - want).abs().max().item()
err_r = (out_r.float() - want).abs().max().item()
print(f"rank {rank}: max |ulysses - full| = {err_u:.4f}, max |ring - full| = {err_r:.4f} (bf16 inputs)")
hdist.destroy_process_group()
dist.destroy_process_group()
