"""Safe settings: a conservative form per kernel family, tried when the tuned form fails its load-time check.

A family whose probe misses its tolerance (or raises) under the tuned settings is given its safe setting - a form
of the same kernel with fewer moving parts - and probed again; if that passes, the family serves with the safe
setting for the life of the process and the verdict line says so (``settings=safe:<families>``).  If the safe form
fails too, the family is refused as before (``KERNELS-REFUSED``, exit 5).  Nothing is ever served by the plain
statements under a kernel mode's label.

| family | tuned | safe |
|---|---|---|
| triattn | four rows per CTA, one exponential in four on the FMA pipe | every exponential on the special-function unit |
| window (atom attention) | tcgen05 kernel, four windows per CTA | CUDA-core kernel, one window per CTA |

Reference: common/opt_core/opt_core/kernels/safe_settings.py (one-stage launch cells when a tuned Triton cell fails
to build).
"""
from __future__ import annotations

from typing import Callable, Dict, List

_ACTIVE: List[str] = []


def _safe_triattn() -> None:
    from . import pair
    pair.set_attention_variant(0x10)


def _safe_window() -> None:
    from . import pair
    pair.WINDOW_KERNEL = "simt"


SAFE: Dict[str, Callable[[], None]] = {"triattn": _safe_triattn, "window": _safe_window}


def apply(family: str) -> bool:
    """Switch ``family`` to its safe setting; False when it has none."""
    fn = SAFE.get(family)
    if fn is None:
        return False
    fn()
    if family not in _ACTIVE:
        _ACTIVE.append(family)
    return True


def active() -> List[str]:
    return list(_ACTIVE)


def word() -> str:
    return "settings=tuned" if not _ACTIVE else "settings=safe:" + ",".join(_ACTIVE)
