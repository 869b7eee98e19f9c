"""One face per op family: ``select()`` is a pure function of (family, sm class, call class, token count, tier word)
over the measured table ``ops/cells.json``; it returns the row that serves and records the decision in the
process-wide cell census.

* tier words: ``fast`` / ``big`` name a kernel row, ``exact`` names the stock statements (bitwise equal to
  ``off``), ``off`` never reaches a provider;
* a call class that the table measured at this token count is a ``cell_hit``; one measured at other counts
  inherits the nearest measured count (``inherited``); a call class outside the table serves the stock statements
  and is counted as ``stock`` with the reason;
* a row can refuse a call by name (``Row.refuses``: head dimension, width, alignment...), in which case the next
  best measured row of the cell is tried and the outcome is ``named_fallback``.

:class:`SizeGate` is the token-count gate in front of a lever with total accounting: every call is counted as
served or as skipped under a reason, so a run's EXIT line can show how much of the work the lever saw.

Reference: kernels/__init__.py:158 (``route``), kernels/triattn/TRIATTN_CELLS.json (``fast_rule``),
attn/size_gate.py:70, common/opt_core/README.md:61-71.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Callable, Dict, Mapping, Optional, Tuple

from ..core import cell_census

TIERS = ("fast", "exact", "big")
_TABLE_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "cells.json")
_TABLE: Optional[dict] = None


def table() -> dict:
    global _TABLE
    if _TABLE is None:
        with open(_TABLE_PATH) as f:
            _TABLE = json.load(f)
    return _TABLE


@dataclass(frozen=True)
class Row:
    family: str
    name: str
    refuses: Optional[Callable[[Mapping], Optional[str]]] = None     # call description -> reason or None


_ROWS: Dict[Tuple[str, str], Row] = {}


def register(row: Row) -> Row:
    _ROWS[(row.family, row.name)] = row
    return row


@dataclass(frozen=True)
class Selection:
    family: str
    row: str                 # the row that serves ("stock" = the plain statements)
    outcome: str             # census outcome word
    key: str                 # table key consulted (or the call's own key when outside the table)
    reason: Optional[str] = None
    expected_ms: Optional[float] = None


def _cells_of(family: str, sm: str, klass: str) -> Dict[int, dict]:
    out = {}
    for key, cell in table().get(family, {}).items():
        s, k, n = key.split("|")
        if s == sm and k == klass:
            out[int(n[1:])] = cell
    return out


def select(family: str, sm: str, klass: str, tokens: int, tier: str, call: Optional[Mapping] = None,
           record: bool = True) -> Selection:
    """Pure over the table: the same arguments give the same row."""
    if tier not in TIERS:
        raise ValueError(f"tier word {tier!r} not in {TIERS}")
    own_key = f"{sm}|{klass}|N{tokens}"
    cells = _cells_of(family, sm, klass)
    if not cells:
        sel = Selection(family, "stock", "stock", own_key, reason=f"call class {klass} not measured on {sm}")
    else:
        n = cell_census.nearest(list(cells), tokens, "ceil")
        cell = cells[n]
        key = f"{sm}|{klass}|N{n}"
        outcome = "cell_hit" if n == tokens else "inherited"
        want = cell["serve"].get(tier, "stock")
        order = [want] + [r for r in cell.get("order", list(cell["rows"])) if r != want]
        sel = None
        first_reason = None
        for name in order:
            if tier == "exact" and name != "stock":
                continue
            row = _ROWS.get((family, name))
            why = row.refuses(call or {}) if (row is not None and row.refuses is not None) else None
            if why is None:
                oc = outcome if name == want else "named_fallback"
                sel = Selection(family, name, oc, key, reason=first_reason, expected_ms=cell["rows"].get(name))
                break
            first_reason = first_reason or f"{name}: {why}"
        if sel is None:
            sel = Selection(family, "stock", "named_fallback", key, reason=first_reason)
    if record:
        # one census entry per call class (its own key); the table cell that answered is the source
        cell_census.record(family, f"{own_key}|{tier}", sel.outcome, row=sel.row, source=f"cells.json:{sel.key}",
                           reason=sel.reason)
    return sel


# rows of this library and what they refuse ---------------------------------------------------------------------
def _needs(**limits):
    def refuses(call: Mapping) -> Optional[str]:
        for k, allowed in limits.items():
            if k in call and call[k] not in allowed:
                return f"{k}={call[k]} (supports {sorted(allowed)})"
        return None
    return refuses


for _name in ("tcgen05_4row", "tcgen05_2row"):
    register(Row("triattn", _name, _needs(head_dim={32, 64}, dtype={"bf16"})))
register(Row("trimul", "tcgen05_3stage", _needs(c_z={128}, c_hidden={128}, dtype={"bf16"})))
register(Row("transition", "tcgen05_fused", _needs(c={128}, expansion={4}, dtype={"bf16"})))
register(Row("transition", "rows_gemm", _needs(dtype={"bf16"})))
register(Row("apb", "tcgen05_2row", _needs(head_dim={32, 64}, dtype={"bf16"})))
register(Row("apb", "tcgen05_window", _needs(head_dim={32}, window={(32, 128)}, dtype={"bf16"})))
register(Row("apb", "simt_window", _needs(head_dim={32}, dtype={"bf16"})))
register(Row("ln", "rows_narrow", _needs(c={64, 128, 256}, dtype={"bf16"})))
register(Row("ln", "rows", None))


@dataclass
class SizeGate:
    """Token-count gate of a lever with total accounting."""
    name: str
    min_tokens: int = 0
    max_tokens: Optional[int] = None
    served: int = 0
    skipped: Dict[str, int] = field(default_factory=dict)

    def admit(self, tokens: int) -> bool:
        if tokens < self.min_tokens:
            why = f"below_min_tokens:{self.min_tokens}"
        elif self.max_tokens is not None and tokens > self.max_tokens:
            why = f"above_max_tokens:{self.max_tokens}"
        else:
            self.served += 1
            return True
        self.skipped[why] = self.skipped.get(why, 0) + 1
        return False

    @property
    def total(self) -> int:
        return self.served + sum(self.skipped.values())

    def words(self) -> str:
        parts = [f"served={self.served}"] + [f"{k}={v}" for k, v in sorted(self.skipped.items())]
        return f"{self.name} total={self.total} " + " ".join(parts)
