"""Census of kernel-provider decisions.

Every time a provider answers "which implementation serves this call class" the decision is
recorded once per key with one of the outcome words ``cell_hit`` (a measured cell of the table),
``inherited`` (nearest measured cell by the inheritance policy), ``named_fallback`` (a declared
refusal; the plain statement serves), ``stock`` (call class outside the table) or ``opt_in``
(forced by the user).  At exit the process prints ``[<tag>] CELLS ...`` lines; a census file can be
summarised from the command line.  Reference: common/opt_core/opt_core/cell_census.py:218,303,439,699.
"""
from __future__ import annotations

import json
import os
import sys
import threading
from typing import Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

from . import report

OUTCOMES = ("cell_hit", "inherited", "named_fallback", "stock", "opt_in")
_LOCK = threading.Lock()
_RECORDS: Dict[Tuple[str, str], dict] = {}


def record(family: str, key: str, outcome: str, row: Optional[str] = None, source: Optional[str] = None,
           reason: Optional[str] = None) -> bool:
    """Record one provider decision; returns True the first time the (family, key) is seen."""
    if outcome not in OUTCOMES:
        raise ValueError(f"census outcome {outcome!r} not in {OUTCOMES}")
    with _LOCK:
        k = (family, key)
        rec = _RECORDS.get(k)
        if rec is None:
            _RECORDS[k] = {"family": family, "key": key, "outcome": outcome, "row": row, "source": source,
                           "reason": reason, "count": 1}
            return True
        rec["count"] += 1
        return False


def records() -> List[dict]:
    with _LOCK:
        return [dict(r) for r in _RECORDS.values()]


def reset() -> None:
    with _LOCK:
        _RECORDS.clear()


def nearest(sizes: Sequence[int], n: int, policy: str = "ceil") -> Optional[int]:
    """Inheritance policy over measured sizes: ``ceil`` = smallest measured size >= n, else the
    largest; ``floor`` = largest measured size <= n, else the smallest; ``closest`` by ratio."""
    if not sizes:
        return None
    s = sorted(sizes)
    if policy == "ceil":
        for x in s:
            if x >= n:
                return x
        return s[-1]
    if policy == "floor":
        for x in reversed(s):
            if x <= n:
                return x
        return s[0]
    if policy == "closest":
        return min(s, key=lambda x: max(x, n) / max(1, min(x, n)))
    raise ValueError(f"unknown inheritance policy {policy!r}")


def summary(recs: Optional[Iterable[Mapping]] = None) -> Dict[str, Dict[str, int]]:
    out: Dict[str, Dict[str, int]] = {}
    for r in (records() if recs is None else recs):
        fam = out.setdefault(r["family"], {o: 0 for o in OUTCOMES})
        fam[r["outcome"]] = fam.get(r["outcome"], 0) + 1
    return out


def exit_lines(tag: str = "opt_core") -> List[str]:
    lines = []
    for fam, counts in sorted(summary().items()):
        lines.append(report.line(tag, "CELLS", ("family", fam), *[(o, counts[o]) for o in OUTCOMES]))
    return lines


def dump(path) -> str:
    with open(path, "w", encoding="utf-8") as f:
        json.dump(records(), f, indent=1, sort_keys=True)
    return str(path)


def install_exit_report(tag: str = "opt_core") -> None:
    env_file = os.environ.get("OPT_CORE_CENSUS_FILE")

    def _line() -> str:
        if env_file:
            try:
                dump(env_file)
            except OSError:
                pass
        ls = exit_lines(tag)
        return "\n".join(ls) if ls else report.line(tag, "CELLS", ("families", 0))

    report.register_exit_tally(tag + ":cells", _line)


def main(argv: Optional[Sequence[str]] = None) -> int:
    """``python -m ...core.cell_census <census.json>``: per-family outcome counts."""
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 1:
        print("usage: cell_census <census.json>", file=sys.stderr)
        return report.EXIT_USAGE
    try:
        with open(argv[0], "r", encoding="utf-8") as f:
            recs = json.load(f)
    except (OSError, ValueError) as e:
        print(f"cannot read {argv[0]}: {e}", file=sys.stderr)
        return report.EXIT_FAIL
    for fam, counts in sorted(summary(recs).items()):
        print(fam, " ".join(f"{o}={counts[o]}" for o in OUTCOMES))
    return report.EXIT_OK


if __name__ == "__main__":
    sys.exit(main())
