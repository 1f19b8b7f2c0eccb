"""Contiguous range sharding of an instruction stream over GPUs / ranks.

Every word decodes independently, so a stream of n words is cut into `world` contiguous
ranges and each rank works on its own range with no exchange step.  Multi-kernel cubins are
cut the same way on the cumulative word count, so a large kernel may span two ranks.
"""
from __future__ import annotations

from typing import Sequence


def shard_range(n: int, world: int, rank: int) -> tuple[int, int]:
    """[begin, end) of rank `rank`: ranges differ in length by at most one word."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    base, extra = divmod(n, world)
    begin = base * rank + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def shard_sections(word_counts: Sequence[int], world: int, rank: int) -> list[tuple[int, int, int]]:
    """Pieces of the sections that fall into rank `rank`'s range of the concatenated stream:
    [(section index, first word inside the section, number of words)]."""
    total = sum(word_counts)
    begin, end = shard_range(total, world, rank)
    out, at = [], 0
    for k, w in enumerate(word_counts):
        lo, hi = max(begin, at), min(end, at + w)
        if lo < hi:
            out.append((k, lo - at, hi - lo))
        at += w
    return out
