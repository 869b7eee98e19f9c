"""The refuse-to-patch rule over a stock function an adapter replaces.

An adapter that wraps or monkey-patches an upstream function was written against one text of that function.
:func:`source_guard` hashes the de-indented source of the function as the running installation has it and
returns a gate: ok when the sha256 is one the adapter names (and every required substring is present), refused
with the observed digest otherwise - a changed upstream is a recorded refusal and the stock function stays in
place.  With neither a digest nor a required text the gate refuses (an unguarded patch is not a guard).
Reference: common/opt_core/opt_core/diffusion_loop/source_guard.py.
"""
from __future__ import annotations

import hashlib
import inspect
import textwrap
from typing import Iterable, Optional

from ..core.gates import Gate


def source_sha256(fn) -> str:
    return hashlib.sha256(textwrap.dedent(inspect.getsource(fn)).encode()).hexdigest()


def source_guard(fn, expected_sha256: Iterable[str] = (), required_text: Iterable[str] = (),
                 name: Optional[str] = None) -> Gate:
    label = name or getattr(fn, "__qualname__", repr(fn))
    expected, required = list(expected_sha256), list(required_text)
    if not expected and not required:
        return Gate(f"source:{label}", False, "no digest and no required text given: an unguarded patch")
    try:
        src = textwrap.dedent(inspect.getsource(fn))
    except (OSError, TypeError) as e:
        return Gate(f"source:{label}", False, f"source unavailable: {e}")
    got = hashlib.sha256(src.encode()).hexdigest()
    if expected and got not in expected:
        return Gate(f"source:{label}", False, f"source digest {got[:16]} is not one the adapter was written for")
    missing = [t for t in required if t not in src]
    if missing:
        return Gate(f"source:{label}", False, f"required text missing: {missing[0][:40]!r}")
    return Gate(f"source:{label}", True, got[:16])
