"""Line protocol and exit rule of a run.

Every process of the framework speaks on stderr in single lines of the form
``[<tag>] <VERB> key=value ...``: ``ACTIVE`` (what engaged), ``NOT ACTIVE: <reason>`` (exit 3,
never a silent fallback), ``LEVER`` (one per optimisation), ``EXIT`` (tally at interpreter
exit).  Exit codes: 0 ok, 1 failed or incomplete, 2 usage, 3 not active or partial, 5 kernels
refused.  Same observable contract as the reference (common/opt_core/opt_core/report.py:39,144,
243,369); the implementation is independent.
"""
from __future__ import annotations

import atexit
import json
import os
import re
import sys
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

EXIT_OK = 0
EXIT_FAIL = 1
EXIT_USAGE = 2
EXIT_NOT_ACTIVE = 3
EXIT_KERNELS_REFUSED = 5

LEVER_STATES = ("on", "off", "skipped")
LEVER_ORIGINS = ("core", "kit")

_WS = re.compile(r"\s+")
_STRATEGY = re.compile(r"(?:F[0-9]+|LOCAL)\.\S+")


def tag_prefix(tag: str) -> str:
    return "[" + tag + "]"


def join(items) -> str:
    """Comma list; ``none`` when empty."""
    if items is None:
        return "none"
    if isinstance(items, (str, bytes)):
        return str(items) or "none"
    items = [str(x) for x in items]
    return ",".join(items) if items else "none"


def _value_text(v) -> str:
    if v is None:
        return "none"
    if isinstance(v, Mapping):
        return ",".join(f"{k}:{x}" for k, x in v.items()) or "none"
    if isinstance(v, (list, tuple, set, frozenset)):
        return join(list(v))
    return str(v)


def kv(*pairs: Tuple[str, object], **fields) -> str:
    """``k=v k2=v2``: positional pairs first (their order is kept), then keywords."""
    seq = list(pairs) + list(fields.items())
    return " ".join(f"{k}={_value_text(v)}" for k, v in seq)


def line(tag: str, verb: str, *pairs, **fields) -> str:
    body = kv(*pairs, **fields)
    head = f"{tag_prefix(tag)} {verb}"
    return head + (" " + body if body else "")


def token(x) -> str:
    """Blank-free text of a value (runs of blanks become ``_``)."""
    s = "none" if x is None else str(x).strip()
    return _WS.sub("_", s) or "none"


def word(key: str, value=None, *parts) -> str:
    """A named evidence word ``key=value(part,...)`` printed on the ACTIVE line: uncertainty a
    lever engaged under (uncertified card, cold cache, safe launch cell).  Never changes the exit code."""
    body = token(value)
    if parts:
        body += "(" + ",".join(token(p) for p in parts) + ")"
    return f"{token(key)}={body}"


def collect_words(*items) -> List[str]:
    out: List[str] = []

    def visit(x):
        if x is None:
            return
        if isinstance(x, str):
            if x and x not in out:
                out.append(x)
            return
        if isinstance(x, Mapping):
            visit(x.get("words"))
            return
        w = getattr(x, "words", None)
        if w is not None:
            visit(list(w() if callable(w) else w))
            return
        for y in x:
            visit(y)

    for it in items:
        visit(it)
    return out


def with_words(text: str, words=None) -> str:
    ws = collect_words(words)
    return text + (" " + " ".join(ws) if ws else "")


def active_line(tag: str, mode: str, levers: Sequence[str] = (), words=None, **fields) -> str:
    return with_words(line(tag, "ACTIVE", ("mode", mode), ("levers", list(levers)), **fields), words)


def not_active_line(tag: str, reason: str, head: Optional[str] = None) -> str:
    return f"{tag_prefix(tag)} NOT ACTIVE: {reason}" + (f" ({head})" if head else "")


def check_strategy(sid: str) -> str:
    if not _STRATEGY.fullmatch(str(sid)):
        raise ValueError(f"strategy id {sid!r} must look like F<k>.<name> or LOCAL.<name>")
    return str(sid)


def lever_line(tag: str, name: str, state: str, *pairs, reason=None, impl=None, origin=None, strategy=None,
               **fields) -> str:
    """``[tag] LEVER name= state= [reason=] impl= origin= [strategy=] evidence...``.

    ``skipped`` requires a reason; ``impl`` and ``origin`` are mandatory; no value may contain blanks.
    """
    if state not in LEVER_STATES:
        raise ValueError(f"lever state {state!r} not in {LEVER_STATES}")
    if state == "skipped" and not reason:
        raise ValueError(f"lever {name!r}: state=skipped needs a reason")
    extra = []
    for k, v in pairs:
        if k in ("name", "state", "reason"):
            raise ValueError(f"{k!r} is positional in lever_line")
        if k == "impl":
            impl = impl if impl is not None else v
        elif k == "origin":
            origin = origin if origin is not None else v
        elif k == "strategy":
            strategy = strategy if strategy is not None else v
        else:
            extra.append((k, v))
    if not impl:
        raise ValueError(f"lever {name!r}: impl is required")
    if origin not in LEVER_ORIGINS:
        raise ValueError(f"lever {name!r}: origin must be one of {LEVER_ORIGINS}")
    head = [("name", name), ("state", state)]
    if reason is not None:
        head.append(("reason", reason))
    head += [("impl", impl), ("origin", origin)]
    if strategy is not None:
        head.append(("strategy", check_strategy(strategy)))
    allp = head + extra + list(fields.items())
    for k, v in allp:
        if any(c.isspace() for c in _value_text(v)):
            raise ValueError(f"lever {name!r}: value of {k!r} contains a blank")
    return line(tag, "LEVER", *allp)


def emit(text: str, stream=None) -> str:
    s = stream if stream is not None else sys.stderr
    s.write(text + "\n")
    s.flush()
    return text


def dump(rep) -> str:
    return json.dumps(rep, indent=1, sort_keys=True, default=str)


def gpu_label(gpu) -> str:
    if isinstance(gpu, Mapping):
        name = gpu.get("name")
        if not name:
            return "none"
        sm = gpu.get("sm") or (("sm" + str(gpu["cc"]).replace(".", "")) if gpu.get("cc") else None)
        if not sm:
            return str(name)
        sm = str(sm)
        return f"{name}({sm if sm.startswith('sm') else 'sm' + sm})"
    return str(gpu) if gpu else "none"


def allow_partial(flag, env_name: str, environ: Optional[Mapping[str, str]] = None) -> bool:
    env = os.environ if environ is None else environ
    return bool(flag) or (env.get(env_name) or "").strip() == "1"


def verdict(rc: int, rep: Optional[Mapping], allow_partial_: bool, incomplete: Optional[str] = None) -> dict:
    """Exit rule of a completed run: incomplete output turns 0 into 1; a partial activation
    (levers of the mode that were not applied) turns 0 into 3 unless allowed; a run that failed
    keeps its own code."""
    rep = rep or {}
    partial = list(rep.get("partial") or [])
    code = int(rc)
    if code == EXIT_OK and incomplete:
        code = EXIT_FAIL
    elif code == EXIT_OK and partial and not allow_partial_:
        code = EXIT_NOT_ACTIVE
    return {"exit_code": code, "partial": partial, "gated": list(rep.get("gated") or []),
            "allow_partial": bool(allow_partial_), "incomplete": incomplete,
            "words": collect_words(rep.get("words"))}


def partial_line(tag: str, v: Mapping, reasons: Optional[Mapping] = None) -> Optional[str]:
    if not v.get("partial"):
        return None
    why = "; ".join(f"{n}: {(reasons or {}).get(n) or 'no reason recorded'}" for n in v["partial"])
    detail = f"levers={join(v['partial'])} ({why})"
    if v.get("allow_partial"):
        return f"{tag_prefix(tag)} PARTIAL allowed: {detail} (--allow-partial, recorded)"
    if v.get("exit_code") == EXIT_NOT_ACTIVE:
        return (f"{tag_prefix(tag)} NOT ACTIVE: partial activation - {detail}; exit {EXIT_NOT_ACTIVE} "
                f"(--allow-partial records and proceeds)")
    return None


# --------------------------------------------------------------------------------- exit tally
IDENTITY_KEYS = ("installed", "armed", "active", "mode", "state", "n_gpu", "rank", "group")
_TALLY: Dict[str, Callable[[], str]] = {}
_PRINTED: set = set()


def tally_fields(stats: Mapping, max_fields: Optional[int] = None, value_chars: int = 40) -> List[str]:
    """``module={k=v,...}`` groups: identity keys first, the rest sorted, omissions named ``...+N``."""
    out = []
    for mod, d in (stats or {}).items():
        if not isinstance(d, Mapping):
            out.append(f"{mod}={_short(d, value_chars)}")
            continue
        ident = [k for k in IDENTITY_KEYS if k in d]
        keys = ident + sorted(k for k in d if k not in ident)
        shown = keys if max_fields is None else keys[:max(0, int(max_fields))]
        parts = []
        for k in shown:
            v = d[k]
            if isinstance(v, Mapping):
                parts.append(f"{k}=<{len(v)}keys>")
            elif isinstance(v, (list, tuple, set, frozenset)):
                parts.append(f"{k}=<{len(v)}items>")
            else:
                parts.append(f"{k}={_short(v, value_chars)}")
        if len(shown) < len(keys):
            parts.append(f"...+{len(keys) - len(shown)}")
        out.append(mod + "={" + ",".join(parts) + "}")
    return out


def _short(v, n):
    s = "none" if v is None else str(v)
    return s if len(s) <= n else s[:max(1, n - 3)] + "..."


def exit_line(tag: str, fields: Optional[str], rc: Optional[int] = None, pid: Optional[int] = None) -> str:
    pid = os.getpid() if pid is None else pid
    head = f"{tag_prefix(tag)} EXIT pid={pid}" + (f" rc={rc}" if rc is not None else "")
    if fields:
        return f"{head} {fields}"
    return f"{head} no lever counters: no lever module was loaded in this process"


def _print_tally(tag: str, fn: Callable[[], str]) -> None:
    if tag in _PRINTED:
        return
    _PRINTED.add(tag)
    try:
        text = fn()
    except Exception as e:  # noqa: BLE001
        text = f"{tag_prefix(tag)} EXIT tally failed: {e!r}"
    try:
        sys.stderr.write(text + "\n")
        sys.stderr.flush()
    except Exception:  # noqa: BLE001
        pass


def register_exit_tally(tag: str, fn: Callable[[], str]) -> bool:
    """Print ``fn()`` once at interpreter exit (a failing ``fn`` prints a tally-failed line)."""
    if tag in _TALLY:
        return False
    _TALLY[tag] = fn
    atexit.register(_print_tally, tag, fn)
    return True


def forced_exit(code: int) -> None:
    """``os._exit`` after printing every registered tally that has not printed yet."""
    for tag, fn in reversed(list(_TALLY.items())):
        _print_tally(tag, fn)
    for s in (sys.stdout, sys.stderr):
        try:
            s.flush()
        except Exception:  # noqa: BLE001
            pass
    os._exit(int(code))
