"""Carry between trunk passes and sample chunking.

``RecycleCarry`` keeps only what the next trunk pass reads (s, z) and drops the rest of a pass;
``sample_chunks`` splits the diffusion samples into chunks that are rolled out one after the other while
drawing the random numbers in the order the unchunked roll-out would (``StockOrderDraws``), so that chunked
and unchunked runs produce the same samples.  Reference: common/opt_core/opt_core/mem/ckpt.py:141,318,399,565,
mem/sample_loop.py:165."""
from __future__ import annotations

from typing import Iterator, List, Tuple

import torch


class RecycleCarry:
    def __init__(self):
        self.s = None
        self.z = None

    def put(self, s, z):
        self.s, self.z = s.detach(), z.detach()

    def take(self):
        s, z = self.s, self.z
        self.s = self.z = None
        return s, z


def sample_chunks(n_samples: int, chunk: int) -> List[Tuple[int, int]]:
    chunk = max(1, min(chunk, n_samples))
    return [(a, min(n_samples, a + chunk)) for a in range(0, n_samples, chunk)]


class StockOrderDraws:
    """Pre-draws the random numbers of an unchunked roll-out step by step ([samples, ...] per draw) and hands
    each chunk its slice, so chunking does not change which numbers a sample sees."""

    def __init__(self, n_samples: int, generator=None, device="cpu"):
        self.n, self.gen, self.device = n_samples, generator, device
        self._cache = {}

    def draw(self, key, shape_per_sample, a: int, b: int) -> torch.Tensor:
        t = self._cache.get(key)
        if t is None:
            t = torch.randn((self.n,) + tuple(shape_per_sample), generator=self.gen, device=self.device)
            self._cache[key] = t
        out = t[a:b]
        if b >= self.n:
            del self._cache[key]
        return out
