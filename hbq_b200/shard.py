"""How the hot path shards across ranks (one process per GPU).

Quantize shards over rows (and over K on block boundaries) with no exchange: every block is
quantised independently, so any split on whole blocks gives the unsharded result.  The GEMM
shards over rows of A (each rank a slice of the batch, W replicated) or over rows of W (column-
parallel; cut on multiples of the partial-sum block ``group_n`` so no quantisation block straddles
ranks).  Neither needs a collective on the data path.
"""
from __future__ import annotations

from typing import Tuple


def row_range(rows: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of ``rows`` owned by ``rank``; sizes differ by at most one."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    q, r = divmod(rows, world)
    begin = rank * q + min(rank, r)
    return begin, begin + q + (1 if rank < r else 0)


def column_range(n: int, rank: int, world: int, multiple: int = 32) -> Tuple[int, int]:
    """[begin, end) of the N output columns owned by ``rank``, cut on multiples of ``multiple``
    (the partial-sum quantisation block) so that every rank owns whole blocks."""
    if n % multiple:
        raise ValueError(f"N={n} is not a multiple of {multiple}")
    b, e = row_range(n // multiple, rank, world)
    return b * multiple, e * multiple


def k_range(k: int, rank: int, world: int, block: int = 128) -> Tuple[int, int]:
    """[begin, end) of K owned by ``rank`` for a K split (row-parallel linear): whole quantisation
    blocks / accumulation groups per rank.  The partial outputs of such a split must then be
    summed across ranks (an all-reduce); that sum is not the reference's sequential fp16 chain,
    so only the fp32 accumulation model keeps its meaning under a K split."""
    if k % block:
        raise ValueError(f"K={k} is not a multiple of {block}")
    b, e = row_range(k // block, rank, world)
    return b * block, e * block
