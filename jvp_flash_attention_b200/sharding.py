"""Batch x head sharding of an attention problem over GPUs.

Every (batch, head) pair is an independent unit in the forward and in the backward pass, so a
multi-GPU run gives each rank a contiguous slice of the flattened B*H axis and needs no
communication on the attention path (the reference's grid axis 1 is exactly Z*H,
jvp_flash_attention/jvp_attention.py:2333-2334).
"""
from __future__ import annotations


def shard_bounds(units: int, world_size: int, rank: int) -> tuple[int, int]:
    """Half-open [lo, hi) slice of ``units`` flattened (b, h) pairs for ``rank``; slices differ by at
    most one unit and cover every unit exactly once."""
    if world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError(f"bad rank {rank} of world size {world_size}")
    base, extra = divmod(units, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def shard_bh(t, world_size: int, rank: int):
    """Slice of a (B, H, N, D) tensor for ``rank`` as a (1, units, N, D) tensor (no copy when contiguous)."""
    B, H = t.shape[:2]
    lo, hi = shard_bounds(B * H, world_size, rank)
    return t.reshape(1, B * H, *t.shape[2:])[:, lo:hi]
