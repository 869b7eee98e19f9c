"""Row layout of the sharded pair tensor.

z[N, N, C] is split by rows: rank p owns rows [r0_p, r1_p).  Shards are as even as possible (the
first N mod P ranks get one more row); ``aligned=True`` rounds shard boundaries to a multiple of
``align`` rows (the 128-row tiles of the fused kernels then never straddle two owners), the last
rank taking the remainder.  Single representation and atoms stay replicated.
Reference: common/opt_core/opt_core/mem/rowpair/API.md (layout section), mem/ngpu.py:35-42.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass(frozen=True)
class Layout:
    n: int          # tokens
    world: int      # ranks
    align: int = 1

    def __post_init__(self):
        if self.world < 1 or self.n < 1:
            raise ValueError("layout needs n >= 1 and world >= 1")

    def bounds(self) -> List[Tuple[int, int]]:
        if self.align <= 1:
            base, rem = divmod(self.n, self.world)
            out, r = [], 0
            for p in range(self.world):
                k = base + (1 if p < rem else 0)
                out.append((r, r + k))
                r += k
            return out
        units = (self.n + self.align - 1) // self.align
        base, rem = divmod(units, self.world)
        out, u = [], 0
        for p in range(self.world):
            k = base + (1 if p < rem else 0)
            out.append((min(u * self.align, self.n), min((u + k) * self.align, self.n)))
            u += k
        return out

    def rows(self, rank: int) -> Tuple[int, int]:
        return self.bounds()[rank]

    def count(self, rank: int) -> int:
        a, b = self.rows(rank)
        return b - a

    def max_count(self) -> int:
        return max(b - a for a, b in self.bounds())

    def owner(self, row: int) -> int:
        for p, (a, b) in enumerate(self.bounds()):
            if a <= row < b:
                return p
        raise IndexError(row)

    def empty_ranks(self) -> List[int]:
        return [p for p, (a, b) in enumerate(self.bounds()) if a == b]
