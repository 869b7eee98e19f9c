"""Batch plans: group sequences by length so that padded batches stay under a token budget and under the
2^31-element ceiling of 32-bit indexing in fused kernels (batch x length x width)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

INT32_ELEMENTS = 2 ** 31 - 1


@dataclass(frozen=True)
class BatchPlan:
    indices: tuple          # positions in the input list
    padded_len: int

    @property
    def tokens(self) -> int:
        return len(self.indices) * self.padded_len


def plan_batches(lengths: Sequence[int], max_tokens: int, width: int = 1, multiple: int = 8,
                 max_batch: int = 1 << 30) -> List[BatchPlan]:
    """Sort by length, then greedily fill batches: padded tokens <= max_tokens and padded elements
    (tokens x width) <= 2^31 - 1.  A single sequence longer than the budget gets a batch of its own."""
    order = sorted(range(len(lengths)), key=lambda i: lengths[i])
    plans: List[BatchPlan] = []
    cur: List[int] = []
    for i in order:
        L = (lengths[i] + multiple - 1) // multiple * multiple
        n = len(cur) + 1
        if cur and (n * L > max_tokens or n * L * width > INT32_ELEMENTS or n > max_batch):
            Lc = (max(lengths[j] for j in cur) + multiple - 1) // multiple * multiple
            plans.append(BatchPlan(tuple(cur), Lc))
            cur = []
        cur.append(i)
    if cur:
        Lc = (max(lengths[j] for j in cur) + multiple - 1) // multiple * multiple
        plans.append(BatchPlan(tuple(cur), Lc))
    return plans
