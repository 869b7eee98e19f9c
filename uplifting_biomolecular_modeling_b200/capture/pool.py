"""When a shape is worth a CUDA-graph capture, and several capture sites under one memory budget.

A policy answers, for a signature the cache has not captured, ``decide(key, sightings) -> (verdict, reason,
final)`` with verdict ``"capture"`` or ``"eager"`` (``final`` files the key as eager for good) and receives the
measured costs of every capture through ``observe`` so that a break-even rule can price the next key.
:class:`GraphPool` holds several :class:`capture.graphs.GraphCache` sites under one byte budget, one item
boundary (``new_item`` drops per-item graphs) and one census.
Reference: common/opt_core/opt_core/capture/pool.py:65 (FixedK), :89 (BreakEven), :132 (Table), :151 (Planned),
:220 (GraphPool).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, Hashable, Mapping, Optional, Tuple

from .graphs import GraphByteBudget, GraphCache


def break_even_k(capture_s: float, saving_s_per_call: float) -> Optional[int]:
    """Calls of one key after which a capture has paid for itself; None when replay saves nothing."""
    if saving_s_per_call <= 0:
        return None
    return max(1, math.ceil(capture_s / saving_s_per_call))


class CapturePolicy:
    """Base policy: capture at first sight."""

    def k(self, key: Hashable) -> Optional[int]:
        return 1

    def decide(self, key: Hashable, sightings: int) -> Tuple[str, str, bool]:
        k = self.k(key)
        if k is None:
            return "eager", "no_row", True
        if sightings >= k:
            return "capture", f"sighting_{sightings}_of_{k}", False
        return "eager", f"sighting_{sightings}_of_{k}", False

    def observe(self, key: Hashable, capture_s: float = 0.0, eager_s: float = 0.0, replay_s: float = 0.0) -> None:
        pass

    # interface of capture.graphs.GraphCache
    def should_capture(self, entry) -> bool:
        return self.decide(getattr(entry, "key", None), entry.calls)[0] == "capture"


class FixedK(CapturePolicy):
    def __init__(self, k: int = 1):
        self._k = int(k)

    def k(self, key):
        return self._k


class BreakEven(CapturePolicy):
    """K from pinned or observed costs: ceil(capture_s / (eager_s - replay_s))."""

    def __init__(self, capture_s: float, saving_s: float):
        self.capture_s, self.saving_s = float(capture_s), float(saving_s)

    def k(self, key):
        return break_even_k(self.capture_s, self.saving_s)

    def observe(self, key, capture_s=0.0, eager_s=0.0, replay_s=0.0):
        if capture_s > 0:
            self.capture_s = capture_s
        if eager_s > 0 and replay_s > 0:
            self.saving_s = eager_s - replay_s


class Table(CapturePolicy):
    """K per key from a pinned table; a key without a row takes ``default_k`` (None: eager, for good)."""

    def __init__(self, rows: Mapping[Hashable, int], default_k: Optional[int] = None):
        self.rows, self.default_k = dict(rows), default_k

    def k(self, key):
        return self.rows.get(key, self.default_k)


class Planned(CapturePolicy):
    """The job declares how many calls of each key it will make; a key is captured at first sight when its
    planned count reaches the break-even K, never otherwise."""

    def __init__(self, counts_by_key: Mapping[Hashable, int], capture_s: float, saving_s: float):
        self.counts = dict(counts_by_key)
        self.need = break_even_k(capture_s, saving_s)

    def k(self, key):
        if self.need is None or self.counts.get(key, 0) < self.need:
            return None
        return 1


@dataclass
class Site:
    name: str
    cache: GraphCache
    per_item: bool = False        # graphs that hold item-specific tensors are dropped at the item boundary
    calls: int = 0
    replays: int = 0


class GraphPool:
    """Capture sites sharing one byte budget and one census."""

    def __init__(self, budget_bytes: Optional[int] = None, default_policy: Optional[CapturePolicy] = None):
        self.budget = GraphByteBudget(budget_bytes) if budget_bytes else None
        self.default_policy = default_policy or FixedK(2)
        self.sites: Dict[str, Site] = {}
        self.items = 0

    def site(self, name: str, policy: Optional[CapturePolicy] = None, per_item: bool = False, **kw) -> Site:
        if name not in self.sites:
            self.sites[name] = Site(name, GraphCache(policy=policy or self.default_policy, budget=self.budget, **kw),
                                    per_item)
        return self.sites[name]

    def call(self, name: str, fn, *args):
        s = self.sites[name]
        s.calls += 1
        before = s.cache.stats["replayed"]
        out = s.cache.run(fn, *args)
        s.replays += s.cache.stats["replayed"] - before
        return out

    def handle(self, name: str) -> "SiteHandle":
        """The site as the object a model calls (``run(fn, *tensors)``, ``stats``, ``words()``): the interface of a
        single :class:`capture.graphs.GraphCache`, counted in this pool's census and held to its byte budget."""
        return SiteHandle(self, name)

    def new_item(self) -> None:
        self.items += 1
        for s in self.sites.values():
            if s.per_item:
                s.cache.entries.clear()

    def census(self) -> Dict[str, Dict[str, int]]:
        return {n: {"calls": s.calls, "replays": s.replays} for n, s in self.sites.items()}


class SiteHandle:
    def __init__(self, pool: GraphPool, name: str):
        self.pool, self.name = pool, name

    def run(self, fn, *tensors):
        return self.pool.call(self.name, fn, *tensors)

    @property
    def stats(self) -> Dict[str, int]:
        return self.pool.sites[self.name].cache.stats

    def words(self):
        return self.pool.sites[self.name].cache.words()
