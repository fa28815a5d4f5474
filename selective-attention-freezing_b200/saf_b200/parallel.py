"""Batch sharding across the GPUs of one box: one process per GPU, replicated weights and patterns,
disjoint batch slices, no collective on the data path (the reference's prefill benchmarks are
single-GPU, and its only multi-GPU mode is data parallelism, nanogpt/train.py:467-472).  The only
communication is the timing reduction (max over ranks) and barriers."""
import os

import torch
import torch.distributed as dist


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def init(backend=None):
    """Initialise the default process group from the torchrun environment (no-op for one process)."""
    rank, world, local = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend=backend, rank=rank, world_size=world, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, world, local


def batch_slice(total_batch, rank, world):
    """[start, stop) of this rank's share of `total_batch` sequences (remainder to the low ranks)."""
    base, rem = divmod(total_batch, world)
    start = rank * base + min(rank, rem)
    return start, start + base + (1 if rank < rem else 0)


def barrier():
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value, device="cpu"):
    """Largest `value` among ranks (timings are reported as the slowest rank's)."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def sum_over_ranks(value, device="cpu"):
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return t.item()


def finalize():
    """Tear the process group down (quietens NCCL's exit warning)."""
    if dist.is_initialized():
        dist.destroy_process_group()
