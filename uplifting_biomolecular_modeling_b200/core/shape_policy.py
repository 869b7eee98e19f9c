"""Padding policies of token counts: kernel tile multiples and the AF3-style size buckets.
Reference: common/opt_core/opt_core/shape_policy.py:27-38."""
from __future__ import annotations

KERNEL_TILE = 64
AF3_BUCKETS = (256, 512, 768, 1024, 1280, 1536, 2048, 2560, 3072, 3584, 4096, 4608, 5120)


def ceil_to(n: int, m: int) -> int:
    return (int(n) + m - 1) // m * m


def pad_to_tile(n: int, tile: int = KERNEL_TILE) -> int:
    return ceil_to(n, tile)


def bucket(n: int, buckets=AF3_BUCKETS) -> int:
    """Smallest bucket >= n; beyond the last bucket, the next multiple of 512."""
    for b in buckets:
        if b >= n:
            return b
    return ceil_to(n, 512)


def plane_leading_dim(n: int) -> int:
    """Leading dimension of channel-major planes: rows must start on 16-byte boundaries for TMA."""
    return ceil_to(n, 8)
