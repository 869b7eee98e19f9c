"""Symmetric peer memory: buffers of equal size on every GPU of the host, each mapped into every rank.

Allocation and handle exchange go through ``torch.distributed._symmetric_memory`` (one process per GPU,
NCCL group for the bootstrap); what the kernels get are raw device pointers of every peer's copy.  The
barrier between "owners wrote their shard" and "peers read it" is this package's own kernel
(``ops/csrc/peer_sm100.cu``): flag words in symmetric memory, system-scope release / acquire, bounded
spin with an error status instead of a hang.  No multimem, no TMA multicast: the kernels read peers with
ordinary TMA / ld.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch

from ..ops import native
from ..ops.native import c_int, c_void_p

native.declare("ubm_peer_barrier", [c_void_p, c_int, c_int, ctypes.c_uint, c_int, c_void_p, c_void_p])
native.declare("ubm_set_flag", [c_void_p, c_int, ctypes.c_uint, c_void_p])


def ptr_array(ptrs: Sequence[int]):
    """Host array of device pointers for the C entry points."""
    arr = (ctypes.c_void_p * len(ptrs))(*[ctypes.c_void_p(int(p)) for p in ptrs])
    return arr


def int_array(vals: Sequence[int]):
    return (ctypes.c_int * len(vals))(*[int(v) for v in vals])


class SymmTensor:
    def __init__(self, local: torch.Tensor, handle, world: int):
        self.local, self.handle, self.world = local, handle, world
        self.ptrs: List[int] = [int(p) for p in handle.buffer_ptrs]

    def ptr(self, rank: int, byte_offset: int = 0) -> int:
        return self.ptrs[rank] + byte_offset

    def peer(self, rank: int, shape, dtype=None, storage_offset: int = 0) -> torch.Tensor:
        return self.handle.get_buffer(rank, tuple(shape), dtype or self.local.dtype, storage_offset)


class SymmHeap:
    """Allocator of symmetric tensors for one process group (all ranks call ``alloc`` in the same order)."""

    def __init__(self, group=None, device: Optional[torch.device] = None):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as sm
        self.sm, self.dist = sm, dist
        self.group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        import warnings
        try:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                sm.enable_symm_mem_for_group(self.group.group_name)
        except Exception:  # noqa: BLE001  (already enabled, or not needed by this torch)
            pass
        self._flags = self.alloc((64,), torch.int32)
        self._flags.local.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)
        self._flag_ptrs = ptr_array(self._flags.ptrs)
        self._epoch = 0
        # Limit of the device-side wait in a stream barrier.  The kernel default (4 s) suits kernels that follow one
        # another on the device; ranks that do host work between steps (checkpoint writes, feature loading) skew by
        # more, so a long-running worker raises it through ROWPAIR_BARRIER_LIMIT_MS (default 60 s).
        self.limit_ms = int(os.environ.get("ROWPAIR_BARRIER_LIMIT_MS", "60000"))

    def alloc(self, shape, dtype) -> SymmTensor:
        t = self.sm.empty(*shape, dtype=dtype, device=self.device)
        h = self.sm.rendezvous(t, self.group)
        return SymmTensor(t, h, self.world)

    def barrier(self, limit_ms: int = 0) -> None:
        """Stream-ordered barrier among the ranks (bounded wait; failure shows in the status word)."""
        self._epoch += 1
        st = native.status_tensor(self.device)
        rc = native.lib().ubm_peer_barrier(self._flag_ptrs, self.rank, self.world, self._epoch,
                                           int(limit_ms) or self.limit_ms,
                                           native.ptr(st), native.current_stream(self.device))
        native.check(rc, "ubm_peer_barrier")
