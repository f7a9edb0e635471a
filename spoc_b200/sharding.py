"""Row-block sharding of the GEMM / map path across the GPUs of one node.

Every output row depends on one row of A and all of B, and maps are
element-independent, so the path shards with no exchange step: rank r owns a
contiguous block of rows of A, C and D (or a contiguous index range of a map);
B and the bias are replicated.  The split rule for sizes that do not divide is
the reference's Vector.partition rule, `base + (i < rem)`
(sarek/core/Vector_storage.ml:261-272).  A gathered result is the
concatenation of the blocks, because row blocks of a row-major matrix are
contiguous.
"""
from __future__ import annotations


def partition(total: int, parts: int) -> list[tuple[int, int]]:
    """[(start, length)] for each part: the first `total % parts` parts get one extra element."""
    if parts <= 0 or total < 0:
        raise ValueError("partition needs parts > 0 and total >= 0")
    base, rem = divmod(total, parts)
    out, start = [], 0
    for i in range(parts):
        n = base + (1 if i < rem else 0)
        out.append((start, n))
        start += n
    return out


def row_block(m: int, world: int, rank: int) -> tuple[int, int]:
    """(first_row, rows) of rank `rank`."""
    return partition(m, world)[rank]


def gather_counts(m: int, n: int, world: int) -> list[int]:
    """Element counts of each rank's block of a row-major m x n result, in rank order."""
    return [rows * n for _, rows in partition(m, world)]
