"""The host-sync census of one sampling step: where a denoising loop makes the CPU wait for the GPU.

:func:`sync_census` runs a callable under torch's CUDA sync debug mode ``"warn"`` and returns the count of
synchronising calls and one record per call site, so that an adapter can name the per-step ``.item()`` /
``.cpu()`` / ``.nonzero()`` sites a sync-free lever would replace and a test can hold a step to a sync count.
The previous debug mode is restored on exit.  A development aid and a regression guard, not a lever.
Reference: common/opt_core/opt_core/diffusion_loop/sync_census.py.
"""
from __future__ import annotations

import warnings
from dataclasses import dataclass, field
from typing import Callable, Dict, List

from ..core.gates import Gate


@dataclass
class SyncSite:
    where: str
    count: int
    text: str


@dataclass
class SyncCensus:
    total: int = 0
    sites: List[SyncSite] = field(default_factory=list)
    result: object = None

    def at_most(self, n: int) -> Gate:
        worst = max(self.sites, key=lambda s: s.count).where if self.sites else "none"
        return Gate("sync_census", self.total <= n, f"{self.total} synchronising calls (limit {n}); busiest {worst}")


def sync_census(fn: Callable[[], object], torch_mod=None) -> SyncCensus:
    torch = torch_mod
    if torch is None:
        import torch  # noqa: PLC0415
    prev = torch.cuda.get_sync_debug_mode() if torch.cuda.is_available() else 0
    if torch.cuda.is_available():
        torch.cuda.set_sync_debug_mode("warn")
    by_site: Dict[str, SyncSite] = {}
    census = SyncCensus()
    try:
        with warnings.catch_warnings(record=True) as caught:
            warnings.simplefilter("always")
            census.result = fn()
        for w in caught:
            if "synchroniz" not in str(w.message).lower():
                continue
            where = f"{w.filename}:{w.lineno}"
            s = by_site.setdefault(where, SyncSite(where, 0, str(w.message)[:120]))
            s.count += 1
            census.total += 1
    finally:
        if torch.cuda.is_available():
            torch.cuda.set_sync_debug_mode(prev)
    census.sites = sorted(by_site.values(), key=lambda s: -s.count)
    return census
