"""Registry behind ``--upstream-fix name[,name...]``: corrections to the stock model that change outputs on
purpose (a bug fix upstream has not released), so they are never part of a mode and must be named by the user.

A fix is a named callable over the model; asking for an unknown name is a usage error that lists the known
ones; every applied fix is reported with a LEVER-style line and recorded in the manifest words, so an output
tree says which stock behaviour it departs from.  Reference: common/opt_core/opt_core/upstream_fix.py.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence

from . import report


class UnknownFix(ValueError):
    pass


@dataclass(frozen=True)
class Fix:
    name: str
    describe: str
    apply: Callable[[object], bool]          # returns False when the model has nothing to fix
    kits: Sequence[str] = ()                 # kits the fix belongs to (empty = any)


_REGISTRY: Dict[str, Fix] = {}


def register(fix: Fix) -> Fix:
    if fix.name in _REGISTRY:
        raise ValueError(f"upstream fix {fix.name!r} registered twice")
    _REGISTRY[fix.name] = fix
    return fix


def known(kit: Optional[str] = None) -> List[str]:
    return sorted(n for n, f in _REGISTRY.items() if not f.kits or kit is None or kit in f.kits)


def parse(arg: Optional[str]) -> List[str]:
    return [] if not arg else [w.strip() for w in arg.split(",") if w.strip()]


def resolve(names: Iterable[str], kit: Optional[str] = None) -> List[Fix]:
    out = []
    for n in names:
        f = _REGISTRY.get(n)
        if f is None or (f.kits and kit is not None and kit not in f.kits):
            raise UnknownFix(f"unknown --upstream-fix {n!r}; known: {', '.join(known(kit)) or 'none'}")
        out.append(f)
    return out


def apply_all(model, names: Iterable[str], tag: str = "opt_core", kit: Optional[str] = None) -> List[str]:
    """Apply the named fixes in the order given; returns the words for the manifest (``fix:<name>`` /
    ``fix:<name>:nothing_to_fix``)."""
    words = []
    for f in resolve(names, kit):
        done = bool(f.apply(model))
        words.append(f"fix:{f.name}" if done else f"fix:{f.name}:nothing_to_fix")
        report.emit(report.line(tag, "UPSTREAM-FIX", ("name", f.name), ("applied", done), ("what", f.describe)))
    return words


def _clear_for_tests() -> None:
    _REGISTRY.clear()
