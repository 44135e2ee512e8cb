"""Batch sharding over the GPUs of one box.

Images are independent and weights read-only, so the forward pass needs no exchange: every rank runs
its own contiguous slice of the batch through its own network instance (the reference does the same
with one OpenMP thread per device, src/DeepNet.cpp:2639-2651).  The only collective is the gather of
the final outputs.  torch.distributed is plumbing here (NCCL on GPUs, gloo in the CPU tests)."""
from __future__ import annotations


def shard_bounds(total: int, world: int, rank: int):
    """[begin, end) of rank's contiguous slice; the first total % world ranks get one more image."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f'rank {rank} outside world {world}')
    base, extra = divmod(total, world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sizes(total: int, world: int):
    return [shard_bounds(total, world, r)[1] - shard_bounds(total, world, r)[0] for r in range(world)]


def gather_outputs(local, total: int, group=None):
    """All-gathers per-rank outputs [n_r][...] (ragged over ranks) into [total][...] on every rank."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    sizes = shard_sizes(total, world)
    width = max(sizes) if sizes else 0
    padded = torch.zeros((width,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: local.shape[0]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)
