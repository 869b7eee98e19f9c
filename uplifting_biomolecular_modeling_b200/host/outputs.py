"""Outputs off the critical path: one bulk device-to-host transfer of a result tree through pinned staging
buffers, then writing in the background.

:func:`to_host` copies every device tensor of a nested dict / list / tuple with non-blocking copies on the
current stream and ONE synchronisation at the end (instead of a blocking ``.cpu()`` per leaf);
:class:`PinnedPool` re-uses page-locked buffers keyed by size; :class:`AsyncWriter` runs ``write(item)`` on
background threads with submit-time ownership of the item, back-pressure (at most ``depth`` pending writes) and
a drain that re-raises the first failure - a lost write is never silent.
Reference: common/opt_core/opt_core/host/outputs.py, host_cache/bg_writer.py.
"""
from __future__ import annotations

import atexit
import concurrent.futures
import sys
import threading
from typing import Any, Callable, Dict, List, Optional

import torch


class PinnedPool:
    """Page-locked host buffers keyed by byte size; ``lease`` hands one out, ``release`` takes it back."""

    def __init__(self, max_bytes: int = 1 << 30):
        self.max_bytes, self.held = max_bytes, 0
        self._free: Dict[int, List[torch.Tensor]] = {}
        self._lock = threading.Lock()
        self.stats = {"leases": 0, "allocs": 0}

    def lease(self, nbytes: int) -> torch.Tensor:
        with self._lock:
            self.stats["leases"] += 1
            lst = self._free.get(nbytes)
            if lst:
                return lst.pop()
            self.stats["allocs"] += 1
            self.held += nbytes
        pin = torch.cuda.is_available()
        return torch.empty(nbytes, dtype=torch.uint8, pin_memory=pin)

    def release(self, buf: torch.Tensor) -> None:
        with self._lock:
            if self.held <= self.max_bytes:
                self._free.setdefault(buf.numel(), []).append(buf)
            else:
                self.held -= buf.numel()


def to_host(tree, pool: Optional[PinnedPool] = None):
    """A copy of ``tree`` with every torch tensor replaced by a CPU tensor; one synchronisation per device."""
    devices = set()

    def walk(x):
        if isinstance(x, torch.Tensor):
            if x.device.type == "cuda":
                devices.add(x.device)
                if pool is not None:
                    buf = pool.lease(x.numel() * x.element_size())
                    host = buf.view(x.dtype).view(x.shape) if x.numel() else torch.empty(x.shape, dtype=x.dtype)
                else:
                    host = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
                host.copy_(x, non_blocking=True)
                return host
            return x.detach().cpu()
        if isinstance(x, dict):
            return {k: walk(v) for k, v in x.items()}
        if isinstance(x, tuple):
            return tuple(walk(v) for v in x)
        if isinstance(x, list):
            return [walk(v) for v in x]
        return x

    out = walk(tree)
    for d in devices:
        torch.cuda.synchronize(d)
    return out


def snapshot(item):
    """An owned copy of ``item`` taken now, in the caller's thread (tensors cloned, containers rebuilt)."""
    if isinstance(item, torch.Tensor):
        return item.detach().clone()
    if isinstance(item, dict):
        return {k: snapshot(v) for k, v in item.items()}
    if isinstance(item, tuple):
        return tuple(snapshot(v) for v in item)
    if isinstance(item, list):
        return [snapshot(v) for v in item]
    return item


class AsyncWriter:
    def __init__(self, write: Callable[[Any], None], workers: int = 1, depth: int = 4, own: bool = True):
        self.write, self.depth, self.own = write, depth, own
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=workers, thread_name_prefix="ubm-writer")
        self._pending: List[concurrent.futures.Future] = []
        self.submitted = self.failed = 0
        self._drained = False
        atexit.register(self._exit_guard)

    def submit(self, item) -> None:
        if self.own:
            item = snapshot(item)
        while len([f for f in self._pending if not f.done()]) >= self.depth:        # back-pressure
            concurrent.futures.wait(self._pending, return_when=concurrent.futures.FIRST_COMPLETED)
        self._pending.append(self._pool.submit(self.write, item))
        self.submitted += 1

    def drain(self) -> int:
        """Wait for every write; re-raise the first failure.  Returns the number of writes."""
        first = None
        for f in self._pending:
            try:
                f.result()
            except BaseException as e:  # noqa: BLE001
                self.failed += 1
                first = first or e
        self._pending.clear()
        self._drained = True
        self._pool.shutdown(wait=True)
        if first is not None:
            raise first
        return self.submitted

    def _exit_guard(self) -> None:
        if not self._drained and self._pending:
            lost = sum(1 for f in self._pending if not f.done() or f.exception() is not None)
            if lost:
                print(f"[ubm-host] WRITER undrained lost={lost} of {self.submitted}", file=sys.stderr)
