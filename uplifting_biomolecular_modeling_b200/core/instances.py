"""Count live instances of a class when activation comes late: a lever that patches a class after some
instances were built must know how many exist (wrap the constructor from now on, seed the count from the
garbage collector once).  Reference: common/opt_core/opt_core/instances.py:136."""
from __future__ import annotations

import gc
import weakref
from typing import Dict, Type


class InstanceCounter:
    def __init__(self, cls: Type):
        self.cls = cls
        self._refs: "weakref.WeakSet" = weakref.WeakSet()
        self.created_after = 0
        self.seeded = 0
        self._orig_init = cls.__init__
        counter = self

        def __init__(obj, *a, **kw):
            counter._orig_init(obj, *a, **kw)
            try:
                counter._refs.add(obj)
            except TypeError:
                pass
            counter.created_after += 1

        cls.__init__ = __init__
        for o in gc.get_objects():
            try:
                if isinstance(o, cls):
                    self._refs.add(o)
                    self.seeded += 1
            except Exception:  # noqa: BLE001
                continue

    def live(self) -> int:
        return len(self._refs)

    def restore(self) -> None:
        self.cls.__init__ = self._orig_init


_COUNTERS: Dict[Type, InstanceCounter] = {}


def track(cls: Type) -> InstanceCounter:
    c = _COUNTERS.get(cls)
    if c is None:
        c = InstanceCounter(cls)
        _COUNTERS[cls] = c
    return c
