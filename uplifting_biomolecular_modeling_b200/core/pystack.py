"""One-off Python-heavy work (a library import, a first launch that builds tables) run away from a stack-chunk edge.

CPython 3.11+ keeps interpreter frames in 16 KiB chunks of a per-thread data stack; a call whose frame does not fit
the current chunk maps a new one and the return that empties it unmaps it again.  A loop that makes one Python call
per iteration while the caller happens to sit at the end of a chunk therefore pays a map / unmap pair per iteration
- microseconds on a plain kernel, tens of microseconds under a system-call-intercepting container runtime, which
turns a one-second import into a minute depending on nothing but the caller's depth.  :func:`roomy_call` runs a
callable from a frame that is itself larger than a chunk: the interpreter gives that frame a chunk of its own size
class and every callee frame lands in the free tail of the same chunk, so no callee starts a chunk.
:func:`call_cost_us` measures the per-call cost at the caller's depth (diagnostic).  Used by :mod:`core.warm` for
its imports.  Reference: common/opt_core/opt_core/_pystack.py:41 (same purpose; there the large frame comes from a
generated source text, here from a code object whose local-variable table is widened with ``code.replace``).
"""
from __future__ import annotations

import sys
import time
from typing import Any, Callable, Optional

SLOTS = 32768          # 8 bytes each: a 256 KiB frame, so the interpreter maps one 512 KiB chunk for the whole call
_ROOMY: Optional[Callable] = None


def _small(fn, args, kwargs):
    return fn(*args, **kwargs)


def _build(slots: int) -> Callable:
    code = _small.__code__
    names = tuple(code.co_varnames) + tuple(f"_pad{i}" for i in range(slots))
    wide = code.replace(co_varnames=names, co_nlocals=len(names))
    import types
    return types.FunctionType(wide, _small.__globals__, "_roomy")


def roomy_call(fn: Callable[..., Any], *args, **kwargs):
    """``fn(*args, **kwargs)`` from the large frame.  Exceptions propagate unchanged; where the large frame cannot be
    built (another interpreter, an older version) the call is made directly."""
    global _ROOMY
    if sys.version_info < (3, 11):
        return fn(*args, **kwargs)
    if _ROOMY is None:
        try:
            _ROOMY = _build(SLOTS)
        except Exception:  # noqa: BLE001 - never cost the caller its call
            _ROOMY = _small
    return _ROOMY(fn, args, kwargs)


def frame_slots() -> int:
    """Local-variable slots of the frame :func:`roomy_call` runs from (0 before its first use)."""
    return 0 if _ROOMY is None else _ROOMY.__code__.co_nlocals


def call_cost_us(n: int = 2000) -> float:
    """Microseconds per trivial Python call at the caller's depth, best of three bursts."""
    def leaf():
        return None
    best = float("inf")
    for _ in range(3):
        t0 = time.perf_counter()
        for _ in range(n):
            leaf()
        best = min(best, (time.perf_counter() - t0) / n * 1e6)
    return best
