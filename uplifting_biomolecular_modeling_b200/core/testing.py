"""Test helpers: run P ranks as threads in one process on the in-process comm backend, golden lines.
Reference: common/opt_core/opt_core/testing.py:28,53,68-109."""
from __future__ import annotations

import threading
import traceback
from typing import Callable, List, Optional


class RankFailure(RuntimeError):
    pass


def run_ranks(world: int, fn: Callable, timeout_s: float = 120.0, hub=None) -> List:
    """Run ``fn(comm)`` on ``world`` rank threads sharing a :class:`parallel.comm.ThreadHub`.  The first
    failing rank aborts the hub (so the others leave their waits); a stuck rank times out.  Returns
    the per-rank results."""
    from ..parallel.comm import ThreadHub
    hub = hub or ThreadHub(world)
    results: List = [None] * world
    errors: List[Optional[str]] = [None] * world

    def body(r: int):
        try:
            results[r] = fn(hub.comm(r))
        except BaseException as e:  # noqa: BLE001
            errors[r] = f"rank {r}: {type(e).__name__}: {e}\n{traceback.format_exc()}"
            hub.abort(f"rank {r} failed: {type(e).__name__}: {e}")

    threads = [threading.Thread(target=body, args=(r,), daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout_s)
    stuck = [i for i, t in enumerate(threads) if t.is_alive()]
    if stuck:
        hub.abort(f"ranks {stuck} stuck after {timeout_s}s")
        raise RankFailure(f"ranks {stuck} did not finish within {timeout_s}s")
    first = next((e for e in errors if e), None)
    if first:
        raise RankFailure(first)
    return results


def golden(lines: List[str], expected: List[str]) -> None:
    """Hold printed lines to recorded ones (pid-like numbers masked)."""
    import re
    mask = lambda s: re.sub(r"pid=\d+", "pid=N", s)  # noqa: E731
    got, want = [mask(x) for x in lines], [mask(x) for x in expected]
    assert got == want, "\n".join(["lines differ:", *("- " + w for w in want), *("+ " + g for g in got)])
