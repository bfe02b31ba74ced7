"""Request-level sharding across GPUs.

Every (request, KV head) segment is independent through the whole decode path, so requests are
simply dealt out to ranks; nothing crosses GPUs on the hot path.  Balance is by total page count
(longest-processing-time-first greedy), which is what the per-step cost is proportional to.
"""
from __future__ import annotations

from typing import List, Sequence


def balance_requests(page_counts: Sequence[int], world_size: int) -> List[List[int]]:
    """Assign request ids to ``world_size`` ranks, heaviest first onto the lightest rank.

    Returns one ascending list of request ids per rank.  Deterministic: ties go to the lower
    request id / lower rank, so every rank computes the same assignment without communication.
    """
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = sorted(range(len(page_counts)), key=lambda i: (-int(page_counts[i]), i))
    load = [0] * world_size
    out: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda k: (load[k], k))
        out[r].append(i)
        load[r] += int(page_counts[i])
    return [sorted(x) for x in out]
