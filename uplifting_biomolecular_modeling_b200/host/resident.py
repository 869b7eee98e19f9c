"""Resident item loop: the model is built and activated once, then a stream of items (inputs on disk, prompts,
batches) runs through it - inputs prepared ahead by a :class:`~host.workers.Prefetcher`, results written behind
by an :class:`~host.outputs.AsyncWriter` - so that per-item cost is the forward pass and not process start-up,
checkpoint load or featurisation.  Reference: common/opt_core/opt_core/host_cache/resident.py.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

from .outputs import AsyncWriter
from .workers import Prefetcher


@dataclass
class ResidentStats:
    items: int = 0
    failed: List[Any] = field(default_factory=list)
    seconds_forward: float = 0.0
    seconds_total: float = 0.0

    def words(self) -> Dict[str, Any]:
        return {"items": self.items, "failed": len(self.failed), "forward_s": round(self.seconds_forward, 3),
                "total_s": round(self.seconds_total, 3)}


def run_resident(items: Iterable[Any], prepare: Callable[[Any], Any], forward: Callable[[Any], Any],
                 write: Callable[[Any], None], workers: int = 1, depth: int = 2,
                 on_error: Optional[Callable[[Any, BaseException], None]] = None) -> ResidentStats:
    """``prepare(item)`` runs on helper threads ahead of the loop, ``forward(prepared)`` on the calling thread (the
    one that owns the device), ``write((item, result))`` on a writer thread behind it.  An item whose preparation
    or forward fails is recorded and skipped (``on_error`` is told); the loop goes on."""
    stats = ResidentStats()
    t_start = time.perf_counter()
    writer = AsyncWriter(write, workers=1, depth=max(2, depth))

    def guarded(item):
        # a failed preparation comes back as a value: the prefetcher's iterator ends at the first exception it raises
        try:
            return True, prepare(item)
        except Exception as e:  # noqa: BLE001
            return False, e

    pf = Prefetcher(guarded, items, workers=workers, depth=depth)
    try:
        for item, (ok, prepared) in pf:
            if not ok:
                stats.failed.append(item)
                if on_error:
                    on_error(item, prepared)
                continue
            t0 = time.perf_counter()
            try:
                result = forward(prepared)
            except Exception as e:  # noqa: BLE001 - one bad item must not end the loop
                stats.failed.append(item)
                if on_error:
                    on_error(item, e)
                continue
            stats.seconds_forward += time.perf_counter() - t0
            writer.submit((item, result))
            stats.items += 1
    finally:
        pf.close()
        writer.drain()
    stats.seconds_total = time.perf_counter() - t_start
    return stats
