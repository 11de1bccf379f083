"""Batch-sharded (data-parallel) execution of a builtin program.

The reference runs every node on devices.front() (ExecutorImpl.cpp:71-75;
ath_device_select, routines.cpp:73-79) and has no collective.  Here each rank
owns one GPU and the rows [rank*B/n, (rank+1)*B/n) of every batch-shaped tensor;
weights are replicated; the only exchange per step is the sum of the weight
gradients over ranks (NCCL all-reduce over NVLink), after which every rank applies
the identical update.  torch.distributed provides the process group.
"""
import os

import torch
import torch.distributed as dist


def shard_rows(global_batch, rank, world):
    """Row range of this rank; the global batch must divide evenly so that every
    rank launches identical shapes."""
    if global_batch % world:
        raise ValueError(f"global batch {global_batch} is not divisible by {world} ranks")
    per = global_batch // world
    return rank * per, (rank + 1) * per


def init_from_env(backend=None):
    """Joins the process group described by RANK/WORLD_SIZE/MASTER_ADDR/MASTER_PORT
    (as torchrun sets them).  Returns (rank, world, local_rank)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, rank=rank, world_size=world,
                                    device_id=torch.device(f"cuda:{local}"))
        else:
            dist.init_process_group(backend, rank=rank, world_size=world)
    return rank, world, local


def make_allreduce(world):
    """Sum over ranks, in place, on the current stream's order."""
    if world <= 1:
        return None

    def allreduce(t):
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t
    return allreduce
