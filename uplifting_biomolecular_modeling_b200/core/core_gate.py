"""Pre-import pin gate of a kit: before the kit imports anything heavy, the shared runtime it was built against is
held to its pin.  A kit calls ``check(tag, pins)`` first thing in its ``__init__``; on a mismatch the process prints
``[<tag>] NOT ACTIVE reason=core_pin ...`` and exits 3 - it never runs half-patched against another runtime.

``pins`` maps a distribution or module name to an exact version (``"1.2.3"``), a prefix (``"1.2.*"``) or a minimum
(``">=1.2"``).  Reference: common/kit_template/_core_gate.py:1-40.
"""
from __future__ import annotations

import sys
from typing import Callable, Mapping, Optional, Tuple

from . import report


def _version_of(name: str) -> Optional[str]:
    try:
        from importlib import metadata
        return metadata.version(name)
    except Exception:
        mod = sys.modules.get(name)
        return getattr(mod, "__version__", None)


def _tuple(v: str) -> Tuple[int, ...]:
    out = []
    for part in v.split("+")[0].split("."):
        digits = "".join(ch for ch in part if ch.isdigit())
        out.append(int(digits) if digits else 0)
    return tuple(out)


def satisfies(version: Optional[str], pin: str) -> bool:
    if version is None:
        return False
    if pin.startswith(">="):
        return _tuple(version) >= _tuple(pin[2:])
    if pin.endswith(".*"):
        return version.split("+")[0].startswith(pin[:-1]) or version.split("+")[0] == pin[:-2]
    return version.split("+")[0] == pin


def mismatches(pins: Mapping[str, str], version_of: Callable[[str], Optional[str]] = _version_of):
    return [(n, p, version_of(n)) for n, p in pins.items() if not satisfies(version_of(n), p)]


def check(tag: str, pins: Mapping[str, str], version_of: Callable[[str], Optional[str]] = _version_of,
          exit_fn: Callable[[int], None] = sys.exit) -> bool:
    bad = mismatches(pins, version_of)
    if not bad:
        return True
    name, pin, got = bad[0]
    report.emit(report.line(tag, "NOT ACTIVE", ("reason", "core_pin"), ("name", name), ("pinned", pin),
                            ("found", got or "missing")))
    exit_fn(report.EXIT_NOT_ACTIVE)
    return False
