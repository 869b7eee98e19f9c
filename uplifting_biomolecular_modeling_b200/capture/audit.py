"""Instruments that decide whether a callable may be captured into a CUDA graph and replayed:

* :class:`LaunchCounter` - kernels of this library launched inside a ``with`` block (entry-point calls, plus the
  kernels accounted to graph replays), by entry point;
* :class:`RNGGuard` - whether the CPU / CUDA generators advanced inside a block (a captured region that draws
  from a generator replays the same numbers unless the draw is made graph-safe);
* :func:`audit_capture_safety` - runs a callable once under the sync census, the RNG guard, the launch counter
  and an allocator probe, and returns an :class:`AuditReport` naming every finding that would break or silently
  change a capture (host synchronisation, generator draws, allocations that grow the reserved pool between two
  warm runs, output that changes between two runs on equal inputs).

Development aids and regression guards, not levers.  Reference: tools/graph_audit/audit.py:1-20 (SyncCensus,
LaunchCounter, RNGGuard, audit_capture_safety).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch

from ..diffusion_loop.sync_census import sync_census
from ..ops import native


class AuditError(AssertionError):
    pass


class LaunchCounter:
    def __init__(self):
        self.before: Dict[str, int] = {}
        self.by_entry: Dict[str, int] = {}

    def __enter__(self) -> "LaunchCounter":
        self.before = native.launch_counts()
        return self

    def __exit__(self, *exc) -> None:
        after = native.launch_counts()
        self.by_entry = {k: v - self.before.get(k, 0) for k, v in after.items() if v - self.before.get(k, 0)}

    @property
    def total(self) -> int:
        return sum(self.by_entry.values())

    @property
    def replays(self) -> int:
        return self.by_entry.get("graph_replay", 0)


def _rng_states(devices) -> List[torch.Tensor]:
    states = [torch.get_rng_state()]
    if torch.cuda.is_available():
        for d in devices:
            states.append(torch.cuda.get_rng_state(d))
    return states


class RNGGuard:
    """``with RNGGuard(expect="unchanged")`` raises :class:`AuditError` when a generator advanced inside the block
    (``expect="advanced"``: when none did; ``expect=None``: only records)."""

    def __init__(self, expect: Optional[str] = None, devices=None):
        if expect not in (None, "unchanged", "advanced"):
            raise ValueError("expect is None, 'unchanged' or 'advanced'")
        self.expect = expect
        self.devices = list(devices) if devices is not None else (
            [torch.cuda.current_device()] if torch.cuda.is_available() else [])
        self.cpu_advanced = False
        self.cuda_advanced = False

    def __enter__(self) -> "RNGGuard":
        self._before = _rng_states(self.devices)
        return self

    def __exit__(self, exc_type, exc, tb) -> None:
        after = _rng_states(self.devices)
        self.cpu_advanced = not torch.equal(self._before[0], after[0])
        self.cuda_advanced = any(not torch.equal(a, b) for a, b in zip(self._before[1:], after[1:]))
        if exc_type is not None:
            return
        if self.expect == "unchanged" and self.advanced:
            raise AuditError("a random generator advanced inside a block that must not draw")
        if self.expect == "advanced" and not self.advanced:
            raise AuditError("no random generator advanced inside a block that must draw")

    @property
    def advanced(self) -> bool:
        return self.cpu_advanced or self.cuda_advanced


@dataclass
class AuditReport:
    syncs: int = 0
    sync_sites: List[str] = field(default_factory=list)
    rng_advanced: bool = False
    launches: Dict[str, int] = field(default_factory=dict)
    pool_growth_bytes: int = 0
    deterministic: bool = True
    findings: List[str] = field(default_factory=list)

    @property
    def safe(self) -> bool:
        return not self.findings

    def line(self, what: str = "region") -> str:
        state = "CAPTURE-SAFE" if self.safe else "NOT-CAPTURE-SAFE"
        return (f"[audit] {what} {state} syncs={self.syncs} rng={'advanced' if self.rng_advanced else 'unchanged'} "
                f"launches={sum(self.launches.values())} pool_growth={self.pool_growth_bytes} "
                f"deterministic={self.deterministic}" + ("" if self.safe else " :: " + "; ".join(self.findings)))


def _flatten(out) -> List[torch.Tensor]:
    if isinstance(out, torch.Tensor):
        return [out]
    if isinstance(out, dict):
        return [t for v in out.values() for t in _flatten(v)]
    if isinstance(out, (list, tuple)):
        return [t for v in out for t in _flatten(v)]
    return []


def audit_capture_safety(fn: Callable[[], object], allow_rng: bool = False, check_determinism: bool = True) -> AuditReport:
    """Run ``fn`` (a zero-argument callable over fixed inputs) three times: a warm-up, then an audited run, then a
    repeat for the determinism and allocator checks.  Nothing is captured; the report says whether capturing it
    would be sound."""
    rep = AuditReport()
    fn()                                                    # warm-up: lazy initialisation is not a finding
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.synchronize()
    reserved0 = torch.cuda.memory_reserved() if cuda else 0
    with LaunchCounter() as lc, RNGGuard() as rg:
        census = sync_census(fn)
    first = [t.detach().clone() for t in _flatten(census.result)]
    rep.syncs, rep.sync_sites = census.total, [f"{s.where} x{s.count}" for s in census.sites]
    rep.rng_advanced, rep.launches = rg.advanced, lc.by_entry
    second = _flatten(fn())
    if cuda:
        torch.cuda.synchronize()
        rep.pool_growth_bytes = max(0, torch.cuda.memory_reserved() - reserved0)
    if check_determinism and not rg.advanced:
        rep.deterministic = len(first) == len(second) and all(
            a.shape == b.shape and torch.equal(a, b) for a, b in zip(first, second))
    if rep.syncs:
        rep.findings.append(f"{rep.syncs} host synchronisation(s): " + ", ".join(rep.sync_sites[:3]))
    if rep.rng_advanced and not allow_rng:
        rep.findings.append("draws from a random generator (a replay would repeat the captured numbers)")
    if rep.pool_growth_bytes:
        rep.findings.append(f"allocator pool grew by {rep.pool_growth_bytes} bytes between two warm runs")
    if not rep.deterministic:
        rep.findings.append("output differs between two runs on equal inputs")
    return rep
