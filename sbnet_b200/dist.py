"""Batch sharding of the block-op pipeline over the GPUs of one node.

Every op of the path is independent per image (a block never crosses images), so the path shards
over batch N with no data-path exchange: one process per GPU, rank r owns a contiguous slice of the
batch and runs reduce_mask -> gather -> ... -> scatter on it with rank-local image indices.  The only
exchange is an all-gather of one int32 per rank -- the per-rank block counts -- which gives the global
block count and each rank's offset in a notional global block list.  The reference has no
counterpart (it is single-GPU); this module is host-side plumbing over ``torch.distributed`` (NCCL
for device tensors, gloo for CPU tests).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_items: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous ``[start, stop)`` slice of ``n_items`` for ``rank``; the first ``n_items % world``
    ranks get one extra item, empty slices are possible when ``world > n_items``."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_items, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def all_gather_counts(count: torch.Tensor, group=None, async_op: bool = False):
    """All-gathers one int32 per rank.  ``count`` is a 1-element int32 tensor (device tensor for NCCL,
    e.g. the device count published by reduce_mask; CPU tensor for gloo).  Returns ``(counts, work)``:
    ``counts`` is an int32 tensor of ``world`` entries, valid once ``work`` (None if synchronous) is
    waited for."""
    world = dist.get_world_size(group)
    out = torch.empty(world, dtype=torch.int32, device=count.device)
    work = dist.all_gather_into_tensor(out, count.reshape(1).to(torch.int32), group=group, async_op=async_op)
    return out, (work if async_op else None)


def block_offsets(counts: Sequence[int]) -> List[int]:
    """Exclusive prefix sum: where each rank's blocks start in the global block list."""
    out, total = [], 0
    for c in counts:
        out.append(total)
        total += int(c)
    return out


def to_global_indices(local_indices: torch.Tensor, count: int, batch_start: int) -> torch.Tensor:
    """Rank-local ``(n, bh, bw)`` triples -> global ones (adds the rank's first image index)."""
    g = local_indices[:count].clone()
    g[:, 0] += batch_start
    return g
