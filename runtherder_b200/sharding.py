"""Row sharding across GPUs.  Every op on the path is row-local (a token row's outputs depend on
that row, the replicated weights and its own position / token id), so rank r of G simply owns the
contiguous block of token rows [floor(r*T/G), floor((r+1)*T/G)) and the matching KV-cache slots;
nothing is exchanged on the data path.  A gather exists for verification only."""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist


def shard_bounds(total_rows: int, world_size: int, rank: int) -> Tuple[int, int]:
    """[begin, end) of rank's row block; blocks are contiguous, cover all rows, differ by at most one."""
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    if total_rows < 0:
        raise ValueError("total_rows must be >= 0")
    return (rank * total_rows) // world_size, ((rank + 1) * total_rows) // world_size


def all_shard_bounds(total_rows: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_bounds(total_rows, world_size, r) for r in range(world_size)]


def gather_rows(local: torch.Tensor, total_rows: int, group=None) -> torch.Tensor:
    """Verification helper: all ranks receive the [total_rows, ...] tensor assembled from the row
    blocks of `shard_bounds` (uneven blocks are padded to the largest for the collective)."""
    world = dist.get_world_size(group)
    bounds = all_shard_bounds(total_rows, world)
    longest = max(e - b for b, e in bounds)
    pad = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    flat = pad.view(torch.uint8) if pad.dtype not in (torch.uint8,) else pad
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat.contiguous(), group=group)
    rows = [p.view(local.dtype).view(pad.shape)[: e - b] for p, (b, e) in zip(parts, bounds)]
    return torch.cat(rows, dim=0)
