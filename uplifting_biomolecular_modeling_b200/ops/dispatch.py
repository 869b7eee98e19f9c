"""Counted kernel dispatch: every call of a switchable module is decided here, before it runs.

A module that a lever switched to its kernel path asks :func:`decide` with the reason (or ``None``) why this
call cannot take the kernel.  The outcome goes into the lever's :class:`~..core.counters.Ledger`
(``served`` / ``fallback:<reason>``) and, once per call class, into the cell census with the row that served
(``cell_hit`` / ``inherited`` when the measured table has the class, ``opt_in`` when the kernel serves a class the
table has not measured, ``named_fallback`` for a plain-statement call).  A fallback reason that the lever did
not declare makes the ledger's ``gate()`` fail at exit, so the run ends ``PARTIAL`` with exit 3 unless the user
passed ``--allow-partial``: a kernel path that quietly ran the plain statements cannot pass as an active mode.

Reference: common/opt_core/opt_core/trimul.py:468 (``Lever.serve``: stock -> below_min -> eligible -> served /
error), common/opt_core/opt_core/counters.py:59, common/opt_core/opt_core/cell_census.py:218.
"""
from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

from ..core import cell_census, counters

# lever -> (implementation word, op family of the provider table, declared fallback reasons)
LEVERS: Dict[str, Tuple[str, str, Tuple[str, ...]]] = {
    "fused_transition": ("transition_sm100@1", "transition", ()),
    "fused_trimul": ("pair_proj+gemm+trimul_out_sm100@1", "trimul", ()),
    "fused_triatt": ("pair_proj+attention_sm100@1", "triattn", ()),
    # keys from another sequence (cross attention) are outside the kernel's call classes by declaration
    "fused_apb": ("attention_sm100@1", "apb", ("cross_keys",)),
    "fused_opm": ("gemm_sm100@1", "opm", ()),
    "fused_pwa": ("gemm_sm100@1", "pwa", ()),
    "fused_dit": ("attention_d64+rows_sm100@1", "apb", ()),
}

_SEEN: set = set()
_SM: Optional[str] = None
TIER = "fast"
# lever -> token-count gate in front of the kernel (the ``below_min`` rung of the reference's ladder).  The kernels
# here serve every size, so the default admits everything; ``UBM_MIN_TOKENS`` / ``UBM_MAX_TOKENS`` (all levers) and
# ``UBM_MIN_TOKENS_<LEVER>`` / ``UBM_MAX_TOKENS_<LEVER>`` set a window, outside of which a call is a DECLARED
# fallback (``below_min_tokens`` / ``above_max_tokens``: counted, named on the lever's line, not PARTIAL).
_GATES: Dict[str, "object"] = {}
SIZE_REASONS = ("below_min_tokens", "above_max_tokens")


def size_gate(lever: str):
    import os
    from . import provider
    g = _GATES.get(lever)
    if g is None:
        def env(word):
            v = os.environ.get(f"UBM_{word}_TOKENS_{lever.upper()}") or os.environ.get(f"UBM_{word}_TOKENS")
            return int(v) if v else None
        g = _GATES[lever] = provider.SizeGate(lever, min_tokens=env("MIN") or 0, max_tokens=env("MAX"))
    return g


def set_tier(word: str) -> None:
    """The tier word of the running mode (``fast`` / ``big``); recorded with every census entry."""
    global TIER
    TIER = word


def _sm() -> str:
    global _SM
    if _SM is None:
        try:
            import torch
            from ..core import arch
            _SM = (arch.device_sm(torch.cuda.current_device()) if torch.cuda.is_available() else None) or "cpu"
        except Exception:  # noqa: BLE001 - the census word only
            _SM = "cpu"
    return _SM


def ledger(lever: str) -> counters.Ledger:
    impl, _, declared = LEVERS.get(lever, ("unknown", lever, ()))
    return counters.BOOK.get(lever, impl, declared_fallbacks=tuple(declared) + SIZE_REASONS,
                             strategy="F1.kernel_fusion")


def decide(lever: str, reason: Optional[str], klass: Optional[str] = None, tokens: Optional[int] = None,
           call: Optional[Mapping] = None, row: Optional[str] = None) -> bool:
    """Record one call.  ``reason`` None = the kernel serves; otherwise the plain statement runs and the call is
    counted as ``fallback:<reason>``.  Returns True when the kernel serves."""
    lg = ledger(lever)
    if reason is None and tokens is not None and not size_gate(lever).admit(int(tokens)):
        reason = "below_min_tokens" if tokens < size_gate(lever).min_tokens else "above_max_tokens"
    if reason is None:
        lg.serve(klass)
    else:
        lg.fallback(reason)
    if klass is not None:
        key = (lever, klass, tokens, reason)
        if key not in _SEEN:
            _SEEN.add(key)
            _census(lever, klass, tokens or 0, reason, call, row)
    return reason is None


def _census(lever, klass, tokens, reason, call, row) -> None:
    from . import provider
    family = LEVERS.get(lever, ("", lever, ()))[1]
    sm = _sm()
    own_key = f"{sm}|{klass}|N{tokens}|{TIER}"
    if reason is not None:
        cell_census.record(family, own_key, "named_fallback", row="stock", source=f"dispatch:{lever}", reason=reason)
        return
    try:
        sel = provider.select(family, sm, klass, tokens, TIER if TIER in provider.TIERS else "fast", call, record=False)
    except Exception:  # noqa: BLE001 - a family without a table is an opt-in class
        sel = None
    if sel is None or sel.row == "stock":
        cell_census.record(family, own_key, "opt_in", row=row or LEVERS[lever][0], source=f"dispatch:{lever}",
                           reason=None if sel is None else sel.reason)
    else:
        cell_census.record(family, own_key, sel.outcome, row=sel.row, source=f"cells.json:{sel.key}", reason=sel.reason)


def reset() -> None:
    """Forget which call classes were recorded and re-read the size windows (tests)."""
    _SEEN.clear()
    _GATES.clear()
