"""Host-side plan of the Ulysses sequence-parallel exchange around an attention call.

Follows the reference's rank group (h3_dit.c:1877-1878, 2529-2546): activations are row-sharded,
``shard_rows = ceil(L / N)`` rows per rank with a zero-padded tail on the last rank; one
head-scatter per tensor gives every rank all rows of ``H / N`` heads; attention runs over the
first L gathered rows only; one sequence-gather returns the output to row shards.
"""
from dataclasses import dataclass


@dataclass(frozen=True)
class UlyssesPlan:
    sequence: int      # L, valid rows of the full sequence
    heads: int         # H
    ranks: int         # N
    shard_rows: int    # rows held by each rank (padded)
    local_heads: int   # heads per rank after the scatter
    padded_rows: int   # shard_rows * ranks, rows of the gathered tensors

    def valid_rows(self, rank):
        """Rows of this rank's shard that carry data (the rest is tail padding)."""
        return max(0, min(self.shard_rows, self.sequence - rank * self.shard_rows))

    def exchange_bytes(self, dim=128, element=2):
        """Bytes one rank sends to its peers in one scatter or gather."""
        return self.shard_rows * self.heads * dim * element * (self.ranks - 1) // self.ranks


def plan(sequence, heads, ranks):
    if ranks < 1 or heads % ranks:
        raise ValueError("Ulysses: %d heads do not split over %d ranks" % (heads, ranks))
    shard_rows = -(-sequence // ranks)
    return UlyssesPlan(sequence, heads, ranks, shard_rows, heads // ranks, shard_rows * ranks)
