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


def boundary_windows(total_rows: int, world_size: int, half_width: int = 64) -> List[Tuple[int, int]]:
    """Row windows [lo, hi) worth checking after a sharded run: the first rows, the last rows, and
    `half_width` rows either side of every shard boundary (merged where they overlap)."""
    cuts = [0] + [e for _, e in all_shard_bounds(total_rows, world_size)]
    spans = sorted((max(0, c - half_width), min(total_rows, c + half_width)) for c in cuts)
    merged: List[Tuple[int, int]] = []
    for lo, hi in spans:
        if hi <= lo:
            continue
        if merged and lo <= merged[-1][1]:
            merged[-1] = (merged[-1][0], max(merged[-1][1], hi))
        else:
            merged.append((lo, hi))
    return merged


def gather_window(local: torch.Tensor, total_rows: int, lo: int, hi: int, group=None) -> torch.Tensor:
    """Verification helper: all ranks receive global rows [lo, hi) of a row-sharded tensor, each row taken
    from the rank that owns it under `shard_bounds` (`local` is this rank's whole row block).  Every rank
    contributes a fixed-size buffer to one all-gather; rows it does not own are left zero and ignored."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bounds = all_shard_bounds(total_rows, world)
    b, e = bounds[rank]
    if local.shape[0] != e - b:
        raise ValueError(f"rank {rank} holds {local.shape[0]} rows, its block is [{b}, {e})")
    n = hi - lo
    mine = torch.zeros((n,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    o_lo, o_hi = max(lo, b), min(hi, e)
    if o_hi > o_lo:
        mine[o_lo - lo:o_hi - lo] = local[o_lo - b:o_hi - b]
    flat = mine.view(torch.uint8) if mine.dtype != torch.uint8 else mine
    parts = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(parts, flat.contiguous(), group=group)
    out = torch.empty_like(mine)
    for p, (rb, re_) in zip(parts, bounds):
        r_lo, r_hi = max(lo, rb), min(hi, re_)
        if r_hi > r_lo:
            out[r_lo - lo:r_hi - lo] = p.view(local.dtype).view(mine.shape)[r_lo - lo:r_hi - lo]
    return out
