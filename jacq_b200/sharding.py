"""Sequence sharding across the GPUs of one box.

The cache-writer / decode-attention path shards by independent sequences: every sequence has its
own block-table row, scratch slot and pages, page pools are per GPU, and no step exchanges data,
so there is no collective on the data path (the reference has none either: its only multi-GPU
mode is a rank-local geometry clone, integrations/vllm_kivi/dsl_decode.py:267-319). What has to be
decided on the host is which rank owns which sequence; for ragged batches the split balances the
bytes each rank must stream rather than the sequence count.
"""
from __future__ import annotations

from typing import Sequence


def contiguous_shards(num_seqs: int, world: int) -> list[range]:
    """Rank r gets a contiguous run; the first ``num_seqs % world`` ranks get one extra."""
    if world <= 0:
        raise ValueError("world must be positive")
    base, extra = divmod(num_seqs, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < extra else 0)
        out.append(range(start, start + n))
        start += n
    return out


def balanced_shards(costs: Sequence[int], world: int) -> list[list[int]]:
    """Longest-processing-time assignment: sequences sorted by cost (e.g. decode bytes) descending,
    each to the currently lightest rank. Deterministic; every sequence appears exactly once."""
    if world <= 0:
        raise ValueError("world must be positive")
    loads = [0] * world
    shards: list[list[int]] = [[] for _ in range(world)]
    for idx in sorted(range(len(costs)), key=lambda i: (-costs[i], i)):
        r = min(range(world), key=lambda j: (loads[j], j))
        shards[r].append(idx)
        loads[r] += costs[idx]
    for s in shards:
        s.sort()
    return shards


def shard_imbalance(costs: Sequence[int], shards: Sequence[Sequence[int]]) -> float:
    """max rank load / mean rank load (1.0 = perfect)."""
    loads = [sum(costs[i] for i in s) for s in shards]
    mean = sum(loads) / max(1, len(loads))
    return max(loads) / mean if mean > 0 else 1.0
