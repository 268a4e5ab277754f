"""Partitioning of the hot path over GPUs: every (batch, kv-head) pair is independent in all three kernels, so the
flattened pairs are block-distributed over the ranks and no collective runs on the data path."""
from __future__ import annotations


def shard_pairs(n_batch: int, n_kv_heads: int, world_size: int, rank: int) -> list[tuple[int, int, int]]:
    """Slices ``(b, h_begin, h_end)`` of the flattened (batch, kv-head) pairs owned by ``rank``; contiguous, disjoint
    over ranks, sizes differing by at most one pair."""
    if not (0 <= rank < world_size):
        raise ValueError(f'rank {rank} outside world of {world_size}')
    total = n_batch * n_kv_heads
    base, extra = divmod(total, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    out = []
    p = lo
    while p < hi:
        b, h = divmod(p, n_kv_heads)
        h_end = min(n_kv_heads, h + (hi - p))
        out.append((b, h, h_end))
        p += h_end - h
    return out


def pairs_per_rank(n_batch: int, n_kv_heads: int, world_size: int) -> list[int]:
    return [sum(h1 - h0 for _, h0, h1 in shard_pairs(n_batch, n_kv_heads, world_size, r)) for r in range(world_size)]
