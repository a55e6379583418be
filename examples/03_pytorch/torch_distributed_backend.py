"""Unmodified torch.distributed code on the "hccl" backend of this library (one process per GPU).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/03_pytorch/torch_distributed_backend.py

Counterpart of HCCL's examples/03_ai_framework/01_pytorch/hccl_pytorch_allreduce_test.py
(dist.init_process_group(backend="hccl") through torch_npu): here importing hccl_b200.torch_backend registers the
backend, and DistributedDataParallel-style gradient averaging runs on HcclAllReduce.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import hccl_b200.torch_backend  # noqa: F401,E402  (registers "hccl")


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("hccl", rank=rank, world_size=world)

    # a data-parallel step by hand: same model everywhere, different data, gradients averaged with all_reduce
    torch.manual_seed(0)
    model = torch.nn.Sequential(torch.nn.Linear(1024, 4096), torch.nn.GELU(), torch.nn.Linear(4096, 1024)).cuda()
    for p in model.parameters():
        dist.broadcast(p.data, src=0)
    opt = torch.optim.SGD(model.parameters(), lr=1e-2)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    for step in range(5):
        x = torch.randn(64, 1024, device="cuda", generator=g)
        loss = model(x).pow(2).mean()
        opt.zero_grad()
        loss.backward()
        for p in model.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step()
        mean_loss = loss.detach().clone()
        dist.all_reduce(mean_loss)
        if rank == 0:
            print(f"step {step}: mean loss {mean_loss.item() / world:.5f}")

    # the parameters stay identical on all ranks
    flat = torch.cat([p.data.reshape(-1) for p in model.parameters()])
    gathered = torch.empty(world * flat.numel(), device="cuda")
    dist.all_gather_into_tensor(gathered, flat)
    same = all(torch.equal(gathered[q * flat.numel():(q + 1) * flat.numel()], flat) for q in range(world))
    if rank == 0:
        print("parameters identical on all ranks:", same)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
