"""Registry of memory levers and the record of an application.

A lever is registered under a name with the hooks it needs from the engine (``Ctx.hooks``) and its
settings (``Ctx.settings``); ``apply(line, ctx)`` applies a comma list of lever names in order and
returns an :class:`AppliedRecord` whose ``active_line`` is the ``mode=big:<levers> refused=<...>`` text of
the kit's ACTIVE line and whose ``gate()`` fails closed when a requested lever was refused without being
declared droppable.  Reference: common/opt_core/opt_core/mem/registry.py:145,201,305, mem/record.py:106,
mem/compose.py:79.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Mapping, Optional, Sequence


class Refusal(RuntimeError):
    """A lever declines to apply; ``kind`` names why, ``fallback`` what serves instead."""

    def __init__(self, kind: str, lever: str = "", fallback: str = "stock"):
        super().__init__(f"{lever or 'lever'} refused: {kind} (fallback {fallback})")
        self.kind, self.lever, self.fallback = kind, lever, fallback


@dataclass
class Ctx:
    hooks: Dict[str, object] = field(default_factory=dict)
    settings: Dict[str, object] = field(default_factory=dict)

    def need(self, name: str):
        if name not in self.hooks:
            raise Refusal(f"hook_missing:{name}")
        return self.hooks[name]


@dataclass
class Lever:
    name: str
    fn: Callable[[Ctx], Optional[dict]]
    label: str = "bitwise"            # bitwise | band (documented tolerance)
    droppable: bool = False
    doc: str = ""


_REGISTRY: Dict[str, Lever] = {}


def register(name: str, label: str = "bitwise", droppable: bool = False):
    def deco(fn):
        _REGISTRY[name] = Lever(name, fn, label, droppable, (fn.__doc__ or "").strip())
        return fn
    return deco


def registered() -> List[str]:
    return sorted(_REGISTRY)


@dataclass
class AppliedRecord:
    base: str = "fast"
    applied: List[str] = field(default_factory=list)
    refused: Dict[str, str] = field(default_factory=dict)
    evidence: Dict[str, dict] = field(default_factory=dict)
    labels: Dict[str, str] = field(default_factory=dict)

    def active_fields(self) -> str:
        exact = all(self.labels.get(n) == "bitwise" for n in self.applied)
        ref = ",".join(f"{k}:{v}" for k, v in self.refused.items()) or "none"
        return f"mode=big:{','.join(self.applied) or 'none'} base={self.base} exact={str(exact).lower()} refused={ref}"

    def gate(self) -> Optional[str]:
        hard = [n for n in self.refused if not (_REGISTRY.get(n) and _REGISTRY[n].droppable)]
        return ("refused:" + ",".join(hard)) if hard else None

    def manifest_block(self) -> dict:
        return {"base": self.base, "applied": list(self.applied), "refused": dict(self.refused),
                "labels": dict(self.labels), "evidence": self.evidence}


def apply(line: str, ctx: Ctx, base: str = "fast") -> AppliedRecord:
    rec = AppliedRecord(base=base)
    for name in [x.strip() for x in line.split(",") if x.strip()]:
        lv = _REGISTRY.get(name)
        if lv is None:
            rec.refused[name] = "unknown_lever"
            continue
        try:
            ev = lv.fn(ctx) or {}
            rec.applied.append(name)
            rec.evidence[name] = ev
            rec.labels[name] = lv.label
        except Refusal as r:
            rec.refused[name] = r.kind
    return rec


def compose_big(table: Mapping[str, Sequence[str]], base: str, levers: Sequence[str] = (), drop: Sequence[str] = (),
                auto: bool = True) -> List[str]:
    """Lever list of ``big``: the base mode's levers plus the memory levers (all registered ones when
    ``auto``), minus ``drop``; order preserved, each once."""
    out: List[str] = []
    for n in list(table.get(base, ())) + (registered() if auto else []) + list(levers):
        if n not in out and n not in drop:
            out.append(n)
    return out
