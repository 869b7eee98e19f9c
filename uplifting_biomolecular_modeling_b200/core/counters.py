"""Per-lever ledgers: every call of a lever is counted as served, as a named fallback, or as an error.

A lever that serves some calls with its own kernel and hands others (by a declared reason) to the
plain statement keeps a :class:`Ledger`; at exit the kit prints the counts on the lever's line and
``gate()`` fails closed when a fallback reason was not declared or an error was recorded, so a
silent degradation cannot pass as an active mode.  Reference: common/opt_core/opt_core/counters.py:59.
"""
from __future__ import annotations

import threading
from typing import Dict, Iterable, Optional, Tuple

from . import report


class Ledger:
    def __init__(self, lever: str, impl: str, origin: str = "core", declared_fallbacks: Iterable[str] = (),
                 strategy: Optional[str] = None, min_tokens: Optional[int] = None):
        self.lever, self.impl, self.origin, self.strategy = lever, impl, origin, strategy
        self.min_tokens = min_tokens
        self.declared = set(declared_fallbacks)
        self.served = 0
        self.fallbacks: Dict[str, int] = {}
        self.errors: Dict[str, int] = {}
        self.shapes: Dict[str, int] = {}
        self._lock = threading.Lock()

    # ---- recording
    def serve(self, shape: Optional[str] = None) -> None:
        with self._lock:
            self.served += 1
            if shape is not None:
                self.shapes[shape] = self.shapes.get(shape, 0) + 1

    def fallback(self, reason: str) -> None:
        with self._lock:
            self.fallbacks[reason] = self.fallbacks.get(reason, 0) + 1

    def error(self, exc: BaseException) -> None:
        with self._lock:
            k = type(exc).__name__
            self.errors[k] = self.errors.get(k, 0) + 1

    # ---- reading
    @property
    def calls(self) -> int:
        return self.served + sum(self.fallbacks.values()) + sum(self.errors.values())

    def undeclared(self) -> Tuple[str, ...]:
        return tuple(sorted(r for r in self.fallbacks if r not in self.declared))

    def gate(self) -> Optional[str]:
        """None when the ledger closes; else the reason the lever counts as not applied."""
        if self.errors:
            return "error:" + ",".join(f"{k}:{v}" for k, v in sorted(self.errors.items()))
        u = self.undeclared()
        if u:
            return "undeclared_fallback:" + ",".join(u)
        if self.calls and not self.served:
            return "never_served"
        return None

    def stats(self) -> dict:
        return {"served": self.served, "fallback": sum(self.fallbacks.values()),
                "fallback_by": dict(sorted(self.fallbacks.items())), "errors": dict(sorted(self.errors.items())),
                "calls": self.calls}

    def line(self, tag: str, state: str = "on", reason: Optional[str] = None) -> str:
        fb = ",".join(f"{k}:{v}" for k, v in sorted(self.fallbacks.items())) or "none"
        fields = [("served", self.served), ("fallback", sum(self.fallbacks.values())), ("fallback_by", fb)]
        if self.min_tokens is not None:
            fields.append(("min_tokens", self.min_tokens))
        if self.shapes:
            top = sorted(self.shapes.items(), key=lambda kv: -kv[1])[:4]
            fields.append(("shapes", ",".join(f"{k}:{v}" for k, v in top)))
        return report.lever_line(tag, self.lever, state, *fields, reason=reason, impl=self.impl, origin=self.origin,
                                 strategy=self.strategy)


class LedgerBook:
    """All ledgers of a process, by lever name."""

    def __init__(self):
        self._ledgers: Dict[str, Ledger] = {}

    def get(self, lever: str, impl: str = "unknown", **kw) -> Ledger:
        lg = self._ledgers.get(lever)
        if lg is None:
            lg = Ledger(lever, impl, **kw)
            self._ledgers[lever] = lg
        return lg

    def items(self):
        return self._ledgers.items()

    def partial(self) -> Dict[str, str]:
        """Levers whose ledger does not close, with the reason."""
        return {n: r for n, lg in self._ledgers.items() for r in [lg.gate()] if r}

    def stats(self) -> dict:
        return {n: lg.stats() for n, lg in self._ledgers.items()}


BOOK = LedgerBook()
