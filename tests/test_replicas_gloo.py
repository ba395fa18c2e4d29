"""Batch sharding across replicas: two gloo ranks on CPU exercise the N > 1 code path (slices, barrier, max-over-ranks
timing) without any GPU or NCCL."""
import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastbb_b200 import replicas


def test_shard_bounds_partition_the_batch():
    for total in (0, 1, 7, 8, 32, 33):
        for world in (1, 2, 4, 8):
            spans = [replicas.shard_bounds(total, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
    assert replicas.shard_bounds(32, 3, 8) == (12, 16)     # ViT-g batch 32 on 8 GPUs: 4 images each


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    r, lr, w = replicas.init_process_group("gloo")
    assert (r, lr, w) == (rank, rank, world)
    batch = torch.arange(10).view(5, 2)
    mine = replicas.local_slice(batch, r, w)
    replicas.barrier()
    slowest = replicas.max_over_ranks(1.0 + rank)            # rank 1 is the slow one
    total = replicas.sum_over_ranks(float(mine.shape[0]))
    per_rank = replicas.gather_over_ranks(10.0 * (rank + 1))
    assert per_rank == [10.0, 20.0]
    gathered = [torch.zeros(3, 2, dtype=batch.dtype) for _ in range(world)]
    pad = torch.zeros(3, 2, dtype=batch.dtype)
    pad[: mine.shape[0]] = mine
    dist.all_gather(gathered, pad)
    if rank == 0:
        out.put((slowest, total, [g.tolist() for g in gathered]))
    dist.destroy_process_group()


def test_two_gloo_ranks_shard_and_reduce():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    slowest, total, gathered = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert slowest == 2.0 and total == 5.0
    assert gathered[0] == [[0, 1], [2, 3], [4, 5]] and gathered[1][:2] == [[6, 7], [8, 9]]


def test_single_process_helpers_are_identities():
    assert replicas.env_rank_world() == (0, 0, 1) or "RANK" in os.environ
    assert replicas.max_over_ranks(3.5) == 3.5 and replicas.sum_over_ranks(2.0) == 2.0
    assert replicas.gather_over_ranks(1.25) == [1.25]
