"""Host parking of pair tensors and streaming through a fixed device window.

``HostPark`` keeps a tensor in pinned host memory; ``stream_blocks`` runs a block function over row blocks
of a parked tensor through two device buffers, prefetching block b+1 on a side stream while block b
computes and writing results back asynchronously.  One ``cudaMemcpyAsync`` per block copy (no batched
memcpy calls).  Reference: common/opt_core/opt_core/mem/offload.py:554,954 and mem/torch_hostpair.py:90-618.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class PinPool:
    """Reusable pinned host buffers keyed by (shape, dtype)."""

    def __init__(self):
        self._free = {}

    def get(self, shape, dtype) -> torch.Tensor:
        key = (tuple(shape), dtype)
        lst = self._free.get(key)
        if lst:
            return lst.pop()
        pin = torch.cuda.is_available()
        return torch.empty(shape, dtype=dtype, pin_memory=pin)

    def put(self, t: torch.Tensor) -> None:
        self._free.setdefault((tuple(t.shape), t.dtype), []).append(t)


class HostPark:
    """A tensor that lives in (pinned) host memory between its uses on the device."""

    def __init__(self, t: torch.Tensor, pool: Optional[PinPool] = None):
        self.shape, self.dtype, self.device = tuple(t.shape), t.dtype, t.device
        self.pool = pool or PinPool()
        self.host = self.pool.get(self.shape, self.dtype)
        self.host.copy_(t, non_blocking=True)
        if t.is_cuda:
            torch.cuda.current_stream(t.device).synchronize()

    def fetch(self, device=None, non_blocking: bool = True) -> torch.Tensor:
        return self.host.to(device or self.device, non_blocking=non_blocking)

    def store(self, t: torch.Tensor) -> None:
        self.host.copy_(t, non_blocking=True)

    def release(self) -> None:
        self.pool.put(self.host)
        self.host = None


def stream_blocks(parked: HostPark, fn: Callable[[torch.Tensor, int, int], torch.Tensor], rows: int,
                  device=None, write_back: bool = True) -> None:
    """Run ``fn(block, a, b)`` over row blocks [a, b) of a parked tensor through a two-buffer device window."""
    dev = torch.device(device) if device is not None else parked.device
    n = parked.shape[0]
    if dev.type != "cuda":
        for a in range(0, n, rows):
            b = min(n, a + rows)
            y = fn(parked.host[a:b], a, b)
            if write_back:
                parked.host[a:b].copy_(y)
        return
    copy_stream = torch.cuda.Stream(dev)
    main = torch.cuda.current_stream(dev)
    bufs = [torch.empty((rows,) + parked.shape[1:], dtype=parked.dtype, device=dev) for _ in range(2)]
    ready = [torch.cuda.Event() for _ in range(2)]
    done = [torch.cuda.Event() for _ in range(2)]
    blocks = [(a, min(n, a + rows)) for a in range(0, n, rows)]

    def prefetch(i):
        a, b = blocks[i]
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(done[i % 2])
            bufs[i % 2][: b - a].copy_(parked.host[a:b], non_blocking=True)
            ready[i % 2].record(copy_stream)

    for e in done:
        e.record(main)
    prefetch(0)
    for i, (a, b) in enumerate(blocks):
        if i + 1 < len(blocks):
            prefetch(i + 1)
        main.wait_event(ready[i % 2])
        y = fn(bufs[i % 2][: b - a], a, b)
        if write_back:
            parked.host[a:b].copy_(y, non_blocking=True)
        done[i % 2].record(main)
    main.synchronize()
