"""Ordered, bounded prefetch: build item k+1 on host workers while the consumer works on item k.

``Prefetcher(build, items, workers=W, depth=D)`` runs ``build(item)`` ahead of the consumer on W threads, keeping
at most D finished-or-running items beyond the one being consumed (host memory is bounded by D feature sets, not
by the input list).  Delivery is in input order; a build that raised re-raises at that item's turn as
:class:`WorkerError` and nothing later is silently skipped.  Reference: common/opt_core/opt_core/host/workers.py.
"""
from __future__ import annotations

import concurrent.futures
import time
from collections import deque
from typing import Any, Callable, Iterable, Iterator, List, Tuple


class WorkerError(RuntimeError):
    def __init__(self, index: int, item: Any, cause: BaseException):
        super().__init__(f"build of item {index} failed: {type(cause).__name__}: {cause}")
        self.index, self.item = index, item
        self.__cause__ = cause


def _timed(build, item):
    t0 = time.perf_counter()
    return build(item), time.perf_counter() - t0


class Prefetcher:
    def __init__(self, build: Callable[[Any], Any], items: Iterable[Any], workers: int = 1, depth: int = 2):
        if workers < 1 or depth < 1:
            raise ValueError("workers and depth must be positive")
        self.build, self.depth = build, depth
        self._items = iter(items)
        self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=workers, thread_name_prefix="ubm-prefetch")
        self._queue: "deque[Tuple[int, Any, concurrent.futures.Future]]" = deque()
        self._next = 0
        self.build_seconds: List[float] = []
        self.waited_seconds = 0.0
        self._closed = False

    def _fill(self) -> None:
        while len(self._queue) < self.depth:
            try:
                item = next(self._items)
            except StopIteration:
                return
            self._queue.append((self._next, item, self._pool.submit(_timed, self.build, item)))
            self._next += 1

    def __iter__(self) -> Iterator[Tuple[Any, Any]]:
        try:
            self._fill()
            while self._queue:
                idx, item, fut = self._queue.popleft()
                self._fill()                      # keep the window full while the consumer waits / works
                t0 = time.perf_counter()
                try:
                    value, secs = fut.result()
                except BaseException as e:  # noqa: BLE001
                    raise WorkerError(idx, item, e) from e
                self.waited_seconds += time.perf_counter() - t0
                self.build_seconds.append(secs)
                yield item, value
        finally:
            self.close()

    def close(self) -> None:
        if not self._closed:
            self._closed = True
            for _, _, fut in self._queue:
                fut.cancel()
            self._pool.shutdown(wait=True)

    def words(self):
        n = len(self.build_seconds)
        return [f"prefetch=items:{n},build_s:{sum(self.build_seconds):.3f},consumer_waited_s:{self.waited_seconds:.3f}"]
