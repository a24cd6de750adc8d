"""Partitioning of the independent (batch, head) problems over the GPUs of one box.

Every (b, h) pair is a self-contained attention problem in forward and backward
(the reference's own launch grid has B*H as an independent axis, flash_attention.py
lines 666, 719, 744), so ranks need no exchange on the data path.  Whole batch
elements are handed out first because they are contiguous in every tensor; heads
are split only when there are more ranks than batch elements.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class BHShard:
    """Half-open ranges of batch elements and heads owned by one rank."""

    b0: int
    b1: int
    h0: int
    h1: int

    @property
    def num_pairs(self) -> int:
        return (self.b1 - self.b0) * (self.h1 - self.h0)

    def slice_bshd(self, t):
        """Slice a (B, S, H, D) tensor."""
        return t[self.b0:self.b1, :, self.h0:self.h1]

    def slice_bhmn(self, t):
        """Slice a (B, H, M, N) tensor."""
        return t[self.b0:self.b1, self.h0:self.h1]


def shard_batch_heads(B: int, H: int, rank: int, world: int) -> BHShard:
    """Returns the (batch, head) block of `rank` among `world` ranks.

    world <= B : B must be divisible by world; each rank gets B/world batch elements.
    world >  B : world must be divisible by B and H by world/B; each rank gets one
                 batch element and H/(world/B) heads.
    """
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    if world <= B:
        if B % world:
            raise ValueError(f"batch {B} is not divisible by {world} ranks")
        per = B // world
        return BHShard(rank * per, (rank + 1) * per, 0, H)
    if world % B:
        raise ValueError(f"{world} ranks is not a multiple of batch {B}")
    groups = world // B
    if H % groups:
        raise ValueError(f"{H} heads cannot be split over {groups} ranks per batch element")
    per = H // groups
    b = rank // groups
    g = rank % groups
    return BHShard(b, b + 1, g * per, (g + 1) * per)
