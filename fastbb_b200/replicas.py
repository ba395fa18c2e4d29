"""Batch sharding for multi-GPU inference: one independent replica of the model per GPU, no collective on the forward
path. Every image is independent (no cross-image operator anywhere in the block stack), so the batch axis is the only
one that shards; the reference itself is single-GPU (README.md:18 "One GPU only").

One process per GPU (torchrun). Each rank keeps a full fp16 copy of the weights, runs its contiguous slice of the batch
and reports its own device time; only that scalar crosses ranks (a MAX all-reduce) when throughput is measured.
"""
import os

import torch
import torch.distributed as dist


def shard_bounds(total, rank, world):
    """[lo, hi) of the contiguous slice of `total` items owned by `rank`: sizes differ by at most one, low ranks first."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def local_slice(x, rank, world, dim=0):
    """This rank's slice of a batch tensor (a view)."""
    lo, hi = shard_bounds(x.shape[dim], rank, world)
    return x.narrow(dim, lo, hi - lo)


def env_rank_world():
    """(rank, local_rank, world_size) from the torchrun environment; (0, 0, 1) when launched as a plain process."""
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def init_process_group(backend=None):
    """Join the torchrun rendezvous if there is one (nccl with GPUs, gloo otherwise); returns (rank, local_rank, world)."""
    rank, local_rank, world = env_rank_world()
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local_rank)
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return rank, local_rank, world


def barrier():
    if dist.is_initialized():
        dist.barrier()


def max_over_ranks(value, device=None):
    """MAX of a Python float over all ranks (identity for a single process)."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or ("cuda" if dist.get_backend() == "nccl" else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(value, device=None):
    """SUM of a Python float over all ranks (identity for a single process)."""
    if not dist.is_initialized():
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or ("cuda" if dist.get_backend() == "nccl" else "cpu"))
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def gather_over_ranks(value, device=None):
    """The Python float of every rank, as a list in rank order (a one-element list for a single process)."""
    if not dist.is_initialized():
        return [float(value)]
    t = torch.tensor([float(value)], dtype=torch.float64, device=device or ("cuda" if dist.get_backend() == "nccl" else "cpu"))
    out = [torch.zeros_like(t) for _ in range(dist.get_world_size())]
    dist.all_gather(out, t)
    return [float(o.item()) for o in out]
