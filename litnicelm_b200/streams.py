"""Partition of independent generation streams over the GPUs of one box.

Streams never exchange data (the reference runs one stream per process,
src/model/inference.cpp:265-296), so the multi-GPU story is a contiguous split
of the stream index range with weights replicated; no collective touches the
data path. Ranks only meet to agree on the slowest rank's time.
"""
from __future__ import annotations

from typing import List, Tuple


def partition_streams(total: int, world: int, rank: int) -> Tuple[int, int]:
    """(first stream, count) of `rank`: contiguous blocks, the first
    total % world ranks carry one extra stream."""
    if world <= 0 or not (0 <= rank < world) or total < 0:
        raise ValueError("bad partition arguments")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    first = rank * base + min(rank, extra)
    return first, count


def all_partitions(total: int, world: int) -> List[Tuple[int, int]]:
    return [partition_streams(total, world, r) for r in range(world)]


def aggregate_tokens_per_s(tokens_per_rank: List[int], seconds_per_rank: List[float]) -> float:
    """Whole-job throughput: all tokens over the slowest rank's time."""
    if not tokens_per_rank or len(tokens_per_rank) != len(seconds_per_rank):
        raise ValueError("per-rank lists must be non-empty and of equal length")
    slowest = max(seconds_per_rank)
    if slowest <= 0:
        raise ValueError("non-positive time")
    return sum(tokens_per_rank) / slowest
