"""Batch sharding of independent sequences over the GPUs of one box (no collective on the data path).

The reference has no multi-GPU mode for this path (N engines on N GPUs); these helpers only decide which
sequences each rank owns.
"""
from __future__ import annotations

import heapq
from typing import Sequence


def shard_even(batch: int, world_size: int, rank: int) -> range:
    """Contiguous, as-even-as-possible split of `batch` sequences; the first batch % world_size ranks get one more."""
    if world_size <= 0 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} / world size {world_size}")
    base, rem = divmod(batch, world_size)
    lo = rank * base + min(rank, rem)
    return range(lo, lo + base + (1 if rank < rem else 0))


def shard_by_tokens(lengths: Sequence[int], world_size: int) -> list[list[int]]:
    """Greedy longest-first assignment of sequences to the least-loaded rank (LPT), balancing token counts.
    Returns, per rank, the sorted indices of its sequences. Deterministic: ties go to the lowest rank / index."""
    if world_size <= 0:
        raise ValueError("world_size must be positive")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    heap = [(0, r) for r in range(world_size)]
    heapq.heapify(heap)
    out: list[list[int]] = [[] for _ in range(world_size)]
    for i in order:
        load, r = heapq.heappop(heap)
        out[r].append(i)
        heapq.heappush(heap, (load + int(lengths[i]), r))
    return [sorted(x) for x in out]
