"""GPU architecture classes and per-lever support declarations.

Levers declare where they are certified (measured), where they may run uncertified, and where they
are excluded; ``supports`` answers with the words ``supported | uncertified | unsupported:<why>`` and
``require`` raises :class:`ArchRefused` (a cannot-run event) so that the mode is refused by name.
This build certifies exactly one class, ``sm100`` (B200): its kernels are tcgen05/TMEM code that no
other class can run.  Reference: common/opt_core/opt_core/arch.py:47,135,186,222,255.
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional, Tuple

from .gates import CannotRun

SM_CLASSES: Dict[str, Dict[str, object]] = {
    "sm80": {"cc": (8, 0), "cards": ("A100",)},
    "sm89": {"cc": (8, 9), "cards": ("L40S", "L4")},
    "sm90": {"cc": (9, 0), "cards": ("H100", "H200")},
    "sm100": {"cc": (10, 0), "cards": ("B200", "GB200")},
    "sm103": {"cc": (10, 3), "cards": ("B300",)},
    "sm120": {"cc": (12, 0), "cards": ("RTX PRO 6000",)},
}

CERTIFIED_DEFAULT = ("sm100",)


class ArchRefused(CannotRun):
    """The lever's mechanism cannot run on this card."""


@dataclass(frozen=True)
class Declaration:
    lever: str
    certified: Tuple[str, ...] = CERTIFIED_DEFAULT
    min_sm: Optional[str] = "sm100"
    exclude: Tuple[str, ...] = ()
    note: str = ""


_DECLS: Dict[str, Declaration] = {}


def sm_number(sm: str) -> int:
    m = re.search(r"(\d+)", str(sm))
    return int(m.group(1)) if m else 0


def sm_of_cc(cc) -> str:
    if isinstance(cc, (tuple, list)):
        return f"sm{cc[0]}{cc[1]}"
    return "sm" + str(cc).replace(".", "")


def declare(lever: str, certified: Iterable[str] = CERTIFIED_DEFAULT, min_sm: Optional[str] = "sm100",
            exclude: Iterable[str] = (), note: str = "") -> Declaration:
    for s in list(certified) + list(exclude) + ([min_sm] if min_sm else []):
        if s not in SM_CLASSES:
            raise ValueError(f"{lever}: unknown sm class {s!r}; known: {', '.join(SM_CLASSES)}")
    d = Declaration(lever, tuple(certified), min_sm, tuple(exclude), note)
    _DECLS[lever] = d
    return d


def declaration(lever: str) -> Optional[Declaration]:
    return _DECLS.get(lever)


def supports(lever: str, sm: str) -> str:
    """``supported`` | ``uncertified`` | ``unsupported:<why>`` for a lever on a card class."""
    d = _DECLS.get(lever)
    if d is None:
        return "uncertified"
    if sm in d.exclude:
        return f"unsupported:excluded_on_{sm}"
    if d.min_sm and sm_number(sm) < sm_number(d.min_sm):
        return f"unsupported:needs_{d.min_sm}"
    if sm in d.certified:
        return "supported"
    return "uncertified"


def require(lever: str, sm: str) -> str:
    """Returns ``supported`` / ``uncertified`` or raises :class:`ArchRefused` naming the lever and the card."""
    v = supports(lever, sm)
    if v.startswith("unsupported"):
        raise ArchRefused(f"lever {lever} cannot run on {sm}: {v.split(':', 1)[1]}")
    return v


def device_sm(index: int = 0) -> Optional[str]:
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        p = torch.cuda.get_device_properties(index)
        return f"sm{p.major}{p.minor}"
    except Exception:  # noqa: BLE001
        return None


def device_memory(index: int = 0) -> Optional[int]:
    """Total device memory in bytes (None without a GPU)."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        return int(torch.cuda.get_device_properties(index).total_memory)
    except Exception:  # noqa: BLE001
        return None


# the levers of this build that are sm_100a machine code
for _name in ("fused_transition", "fused_trimul", "fused_triatt", "fused_apb", "fused_opm", "fused_pwa",
              "fused_dit", "rowpair_fused", "tp_fused"):
    declare(_name, certified=("sm100",), min_sm="sm100", note="tcgen05/TMEM/TMA kernels")
