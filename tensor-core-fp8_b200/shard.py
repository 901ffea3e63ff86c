"""N-sharded multi-GPU plan for one large GEMM.

C's columns are independent and B is stored as N rows of K bytes, so a column block of
B / C is a contiguous row slab of B's storage: rank r of R owns rows
[n_begin, n_end) of B and the same columns of C; A is replicated.  The compute step
exchanges nothing.  An all-gather of the C blocks is optional and timed separately.
(The reference has no multi-GPU code; its operator, GEMM/include/gemm.cuh:12-55, is
what each rank calls on its shard.)
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class Shard:
    rank: int
    world: int
    n_begin: int
    n_end: int

    @property
    def n(self) -> int:
        return self.n_end - self.n_begin


def column_shard(n: int, rank: int, world: int, align: int = 256) -> Shard:
    """Even split of N columns in units of `align` (the widest tile), remainder to the low ranks."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError("bad rank/world")
    units = (n + align - 1) // align
    base, extra = divmod(units, world)
    begin_u = rank * base + min(rank, extra)
    end_u = begin_u + base + (1 if rank < extra else 0)
    return Shard(rank, world, min(n, begin_u * align), min(n, end_u * align))


def all_shards(n: int, world: int, align: int = 256):
    return [column_shard(n, r, world, align) for r in range(world)]


def gather_layout_to_row_major(blocks, m: int):
    """All-gather returns [R][M][N/R]; this is the index map back to row-major [M][N] (host-side check)."""
    import torch
    return torch.cat([b.reshape(m, -1) for b in blocks], dim=1)
