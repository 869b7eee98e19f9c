"""Host-side memory primitives of ``big`` mode.

* :class:`HostChunks` - a pool of pinned host chunks whose sizes are powers of two: a request is served by the
  smallest free chunk that fits, so a run with many slightly different sizes pins a bounded set of buffers.
* :class:`HostPair` - a pair tensor ``[N, N, C]`` that lives in pinned host memory and is visited through a device
  window of ``rows`` rows: ``rows(i0, i1)`` brings a row block in, ``cols(j0, j1)`` a column block (strided host
  read, contiguous on the device), ``put_rows`` writes a block back.
* :class:`LayerNormGuard` - LayerNorm over tensors of 2^31 elements or more, applied in row chunks below the
  limit (library LayerNorm kernels index with 32-bit integers).

Reference: common/opt_core/opt_core/mem/torch_hostpair.py:90,325,460,618.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F

INT32_ELEMENTS = 2 ** 31


def _pow2_at_least(n: int) -> int:
    return 1 << max(0, (int(n) - 1).bit_length())


class HostChunks:
    def __init__(self, min_bytes: int = 1 << 20, pin: Optional[bool] = None):
        self.min_bytes = int(min_bytes)
        self.pin = torch.cuda.is_available() if pin is None else pin
        self._free: Dict[int, List[torch.Tensor]] = {}
        self.allocated_bytes = 0
        self.leases = 0

    def lease(self, nbytes: int) -> torch.Tensor:
        """A uint8 buffer of at least ``nbytes`` (its size is a power of two, at least ``min_bytes``)."""
        size = max(self.min_bytes, _pow2_at_least(nbytes))
        self.leases += 1
        lst = self._free.get(size)
        if lst:
            return lst.pop()
        self.allocated_bytes += size
        return torch.empty(size, dtype=torch.uint8, pin_memory=self.pin)

    def release(self, buf: torch.Tensor) -> None:
        self._free.setdefault(buf.numel(), []).append(buf)

    def view(self, buf: torch.Tensor, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return buf[:nbytes].view(dtype).view(*shape)


class HostPair:
    def __init__(self, N: int, C: int, dtype=torch.bfloat16, device="cpu", chunks: Optional[HostChunks] = None):
        self.N, self.C, self.dtype, self.device = N, C, dtype, torch.device(device)
        self.chunks = chunks or HostChunks()
        self._buf = self.chunks.lease(N * N * C * torch.empty((), dtype=dtype).element_size())
        self.host = self.chunks.view(self._buf, (N, N, C), dtype)

    @classmethod
    def from_tensor(cls, z: torch.Tensor, chunks: Optional[HostChunks] = None) -> "HostPair":
        hp = cls(z.shape[0], z.shape[2], z.dtype, z.device, chunks)
        hp.host.copy_(z)
        return hp

    def rows(self, i0: int, i1: int) -> torch.Tensor:
        return self.host[i0:i1].to(self.device, non_blocking=True)

    def cols(self, j0: int, j1: int) -> torch.Tensor:
        """Column block [N, j1 - j0, C]: a strided read on the host, contiguous on the device."""
        return self.host[:, j0:j1].contiguous().to(self.device, non_blocking=True)

    def put_rows(self, i0: int, block: torch.Tensor) -> None:
        self.host[i0:i0 + block.shape[0]].copy_(block, non_blocking=True)

    def map_rows(self, fn, rows: int) -> None:
        """z[i0:i1] = fn(z[i0:i1], i0, i1) block by block through the device window."""
        for i0 in range(0, self.N, rows):
            i1 = min(self.N, i0 + rows)
            self.put_rows(i0, fn(self.rows(i0, i1), i0, i1))
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    def release(self) -> None:
        self.chunks.release(self._buf)
        self.host = None


class LayerNormGuard:
    """``guard(x, weight, bias, eps)`` = LayerNorm over the last dimension, in row chunks when ``x`` has 2^31
    elements or more (``limit`` is a parameter so that the chunked path can be exercised on small tensors)."""

    def __init__(self, limit: int = INT32_ELEMENTS):
        self.limit = limit
        self.chunked_calls = 0

    def __call__(self, x: torch.Tensor, weight, bias, eps: float = 1e-5) -> torch.Tensor:
        C = x.shape[-1]
        if x.numel() < self.limit:
            return F.layer_norm(x, (C,), weight, bias, eps)
        self.chunked_calls += 1
        flat = x.reshape(-1, C)
        rows = max(1, (self.limit - 1) // C)
        out = torch.empty_like(flat)
        for r0 in range(0, flat.shape[0], rows):
            out[r0:r0 + rows] = F.layer_norm(flat[r0:r0 + rows], (C,), weight, bias, eps)
        return out.view(x.shape)
