"""Batch sharding across the GPUs of one box.

Images are independent (the reference evaluates one image per call), so a batch
is split into contiguous chunks, one per rank, with no collective on the data
path.  Only when the caller wants every output on every rank are the per-rank
results gathered (NCCL over NVLink on GPUs; the same code runs on gloo for tests).
"""
from __future__ import annotations


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous chunk [begin, end) of `total` images for `rank`: ceil(total/world) each,
    the last ranks may receive fewer (or none)."""
    if total < 0 or world <= 0 or not 0 <= rank < world:
        raise ValueError("invalid shard request")
    per = -(-total // world)
    begin = min(rank * per, total)
    return begin, min(begin + per, total)


def gather_outputs(local, total: int, group=None):
    """All-gathers per-rank output chunks (torch tensors [n_local, ...]) into [total, ...].
    Chunks may be ragged; they are padded to the largest chunk for the collective."""
    import torch
    import torch.distributed as dist

    world = dist.get_world_size(group)
    per = -(-total // world)
    padded = local
    if local.shape[0] < per:
        pad = torch.zeros((per - local.shape[0], *local.shape[1:]), dtype=local.dtype, device=local.device)
        padded = torch.cat([local, pad], 0)
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded.contiguous(), group=group)
    return torch.cat(parts, 0)[:total]
