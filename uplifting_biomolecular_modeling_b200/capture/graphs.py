"""CUDA-graph cache keyed by the signature of a call.

``GraphCache.run(fn, *tensors)``: the first ``eager_first`` calls of a signature run eagerly (kernels
compile, workspaces get allocated); the next call captures ``fn`` on static copies of the inputs; later
calls copy the inputs in and replay.  With ``verify >= 1`` the first replays are compared bit for bit with an
eager run of the same inputs and a mismatch retires the graph for that signature.  A failed capture is
recorded, the stream is left usable and the signature falls back to eager for good.  A byte budget caps the
memory held by captured graphs' static buffers.  Reference: common/opt_core/opt_core/capture/graphs.py:494,515,569
and capture/pool.py:65-220.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch


def signature(tensors) -> Tuple:
    return tuple((tuple(t.shape), str(t.dtype), str(t.device)) if isinstance(t, torch.Tensor) else ("py", repr(t))
                 for t in tensors)


class GraphByteBudget:
    def __init__(self, limit_bytes: int):
        self.limit, self.used = int(limit_bytes), 0

    def admit(self, nbytes: int) -> bool:
        if self.used + nbytes > self.limit:
            return False
        self.used += nbytes
        return True


@dataclass
class _Entry:
    calls: int = 0
    graph: Optional["torch.cuda.CUDAGraph"] = None
    static_in: Optional[List[torch.Tensor]] = None
    static_out: object = None
    retired: Optional[str] = None
    verified: int = 0
    replays: int = 0


class FixedK:
    """Capture after K eager calls of a signature."""

    def __init__(self, k: int = 1):
        self.k = k

    def should_capture(self, entry: _Entry) -> bool:
        return entry.calls > self.k


class BreakEven:
    """Capture once the signature has recurred often enough to pay for the capture."""

    def __init__(self, capture_cost_calls: float = 3.0):
        self.cost = capture_cost_calls

    def should_capture(self, entry: _Entry) -> bool:
        return entry.calls > self.cost


class GraphCache:
    def __init__(self, policy=None, verify: int = 1, budget: Optional[GraphByteBudget] = None,
                 enabled: Optional[bool] = None):
        self.policy = policy or FixedK(1)
        self.verify = verify
        self.budget = budget
        self.enabled = torch.cuda.is_available() if enabled is None else enabled
        self.entries: Dict[Tuple, _Entry] = {}
        self.stats = {"eager": 0, "captured": 0, "replayed": 0, "retired": 0, "capture_failed": 0}

    def words(self) -> List[str]:
        return [f"graphs=captured:{self.stats['captured']},retired:{self.stats['retired']}"]

    def run(self, fn: Callable, *tensors):
        if not self.enabled:
            self.stats["eager"] += 1
            return fn(*tensors)
        key = signature(tensors)
        e = self.entries.setdefault(key, _Entry())
        e.calls += 1
        if e.retired is not None or (e.graph is None and not self.policy.should_capture(e)):
            self.stats["eager"] += 1
            return fn(*tensors)
        if e.graph is None:
            self._capture(e, fn, tensors)
            if e.graph is None:
                self.stats["eager"] += 1
                return fn(*tensors)
        for s, t in zip(e.static_in, tensors):
            if isinstance(t, torch.Tensor):
                s.copy_(t)
        e.graph.replay()
        e.replays += 1
        self.stats["replayed"] += 1
        out = _clone_tree(e.static_out)
        if e.verified < self.verify:
            ref = fn(*tensors)
            e.verified += 1
            if not _equal_tree(ref, out):
                e.retired = "replay_differs_from_eager"
                self.stats["retired"] += 1
                return ref
        return out

    def _capture(self, e: _Entry, fn, tensors) -> None:
        nbytes = sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))
        if self.budget is not None and not self.budget.admit(nbytes):
            e.retired = "byte_budget"
            self.stats["retired"] += 1
            return
        try:
            static_in = [t.clone() if isinstance(t, torch.Tensor) else t for t in tensors]
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn(*static_in)
            torch.cuda.current_stream().wait_stream(side)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = fn(*static_in)
            e.graph, e.static_in, e.static_out = g, static_in, out
            self.stats["captured"] += 1
        except Exception as ex:  # noqa: BLE001
            e.retired = f"capture_failed:{type(ex).__name__}"
            self.stats["capture_failed"] += 1
            torch.cuda.synchronize()


def _clone_tree(x):
    if isinstance(x, torch.Tensor):
        return x.clone()
    if isinstance(x, (list, tuple)):
        return type(x)(_clone_tree(y) for y in x)
    if isinstance(x, dict):
        return {k: _clone_tree(v) for k, v in x.items()}
    return x


def _equal_tree(a, b) -> bool:
    if isinstance(a, torch.Tensor):
        return isinstance(b, torch.Tensor) and torch.equal(a, b)
    if isinstance(a, (list, tuple)):
        return len(a) == len(b) and all(_equal_tree(x, y) for x, y in zip(a, b))
    if isinstance(a, dict):
        return a.keys() == b.keys() and all(_equal_tree(a[k], b[k]) for k in a)
    return a == b
