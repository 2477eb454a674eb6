"""Position sharding for multi-GPU runs.

Positions are independent (the batch is the leading dimension of every buffer of the
reference graph, network.py:328-340), so each GPU takes one contiguous range and there is no
collective on the data path.
"""

from __future__ import annotations


def shard_range(total: int, rank: int, world: int) -> tuple[int, int]:
    """Half-open range of positions for ``rank`` of ``world``; sizes differ by at most one."""
    if total < 0 or world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad shard request: total={total} rank={rank} world={world}")
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)
