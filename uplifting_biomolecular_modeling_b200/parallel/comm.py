"""One communication surface for every sharded schedule.

No schedule calls ``torch.distributed`` itself; it gets a :class:`Comm` with the handful of collectives
the row-sharded pair stack needs, and three interchangeable backends:

* ``SoloComm``   - world 1, every collective is the identity (P = 1 equals the dense statement),
* ``ThreadComm`` - P rank *threads* in one process exchanging through a :class:`ThreadHub` (CPU tests
                   of the schedules without a cluster),
* ``GroupComm``  - a ``torch.distributed`` process group (NCCL on CUDA, gloo on CPU).

Host-side signalling (``host_signal`` / ``host_wait``) goes through a key-value store so that an idle
rank waits on the CPU with a timeout, never inside a posted collective.
Reference: common/opt_core/opt_core/mem/rowpair/dist.py:380,610,733,834,923.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional, Sequence

import torch


class CommAborted(RuntimeError):
    """Another rank failed, or a wait ran past its limit."""


class Comm:
    rank: int = 0
    world: int = 1
    backend: str = "solo"

    # -- collectives (all ranks call in the same order)
    def all_gather(self, t: torch.Tensor) -> List[torch.Tensor]:
        raise NotImplementedError

    def all_to_all(self, parts: Sequence[torch.Tensor]) -> List[torch.Tensor]:
        """parts[q] goes to rank q; returns what every rank sent to this one."""
        raise NotImplementedError

    def broadcast(self, t: torch.Tensor, src: int = 0) -> torch.Tensor:
        raise NotImplementedError

    def all_reduce_scalar(self, v: float, op: str = "max") -> float:
        raise NotImplementedError

    def barrier(self) -> None:
        raise NotImplementedError

    # -- host-side store
    def host_signal(self, key: str, value: str = "1") -> None:
        raise NotImplementedError

    def host_wait(self, key: str, timeout_s: float = 60.0) -> str:
        raise NotImplementedError

    # -- helpers built on the above
    def all_gather_rows(self, t: torch.Tensor) -> torch.Tensor:
        """Concatenate row shards (dimension 0) of possibly different lengths."""
        return torch.cat(self.all_gather(t), dim=0)

    def gather_to(self, t: torch.Tensor, dst: int = 0) -> Optional[torch.Tensor]:
        parts = self.all_gather(t)
        return torch.cat(parts, 0) if self.rank == dst else None

    def check_replicated(self, t: torch.Tensor, what: str = "tensor") -> None:
        """Refuse by name when a tensor that must be identical on all ranks is not."""
        s = float(t.double().sum().item()) if t.numel() else 0.0
        lo, hi = self.all_reduce_scalar(s, "min"), self.all_reduce_scalar(s, "max")
        if lo != hi:
            raise CommAborted(f"replication guard: {what} differs across ranks (checksum {lo} .. {hi})")


class SoloComm(Comm):
    def __init__(self):
        self.rank, self.world, self.backend = 0, 1, "solo"
        self._store: Dict[str, str] = {}

    def all_gather(self, t):
        return [t]

    def all_to_all(self, parts):
        return [parts[0]]

    def broadcast(self, t, src=0):
        return t

    def all_reduce_scalar(self, v, op="max"):
        return v

    def barrier(self):
        return None

    def host_signal(self, key, value="1"):
        self._store[key] = value

    def host_wait(self, key, timeout_s=60.0):
        if key not in self._store:
            raise CommAborted(f"host_wait({key}): never signalled")
        return self._store[key]


# ---------------------------------------------------------------------------- threads
class ThreadHub:
    """Rendezvous of P rank threads.  Every collective is an exchange through a slot table guarded by a
    condition variable; ``abort`` wakes all waiters with :class:`CommAborted`."""

    def __init__(self, world: int, timeout_s: float = 60.0):
        self.world, self.timeout_s = world, timeout_s
        self._cv = threading.Condition()
        self._slots: Dict[int, Dict[int, object]] = {}
        self._done: Dict[int, int] = {}
        self._aborted: Optional[str] = None
        self._store: Dict[str, str] = {}
        self._seq = [0] * world

    def comm(self, rank: int) -> "ThreadComm":
        return ThreadComm(self, rank)

    def abort(self, why: str) -> None:
        with self._cv:
            if self._aborted is None:
                self._aborted = why
            self._cv.notify_all()

    def exchange(self, rank: int, payload) -> Dict[int, object]:
        """All ranks deposit a payload under the same sequence number and get everybody's back."""
        seq = self._seq[rank]
        self._seq[rank] += 1
        deadline = time.time() + self.timeout_s
        with self._cv:
            self._slots.setdefault(seq, {})[rank] = payload
            self._cv.notify_all()
            while len(self._slots[seq]) < self.world:
                if self._aborted:
                    raise CommAborted(self._aborted)
                left = deadline - time.time()
                if left <= 0:
                    self._aborted = f"rank {rank}: collective #{seq} timed out after {self.timeout_s}s"
                    self._cv.notify_all()
                    raise CommAborted(self._aborted)
                self._cv.wait(min(left, 0.5))
            if self._aborted:
                raise CommAborted(self._aborted)
            out = dict(self._slots[seq])
            self._done[seq] = self._done.get(seq, 0) + 1
            if self._done[seq] == self.world:
                del self._slots[seq]
                del self._done[seq]
            return out

    def signal(self, key, value):
        with self._cv:
            self._store[key] = value
            self._cv.notify_all()

    def wait(self, key, timeout_s):
        deadline = time.time() + timeout_s
        with self._cv:
            while key not in self._store:
                if self._aborted:
                    raise CommAborted(self._aborted)
                left = deadline - time.time()
                if left <= 0:
                    raise CommAborted(f"host_wait({key}) timed out after {timeout_s}s")
                self._cv.wait(min(left, 0.5))
            return self._store[key]


class ThreadComm(Comm):
    def __init__(self, hub: ThreadHub, rank: int):
        self.hub, self.rank, self.world, self.backend = hub, rank, hub.world, "threads"

    def all_gather(self, t):
        got = self.hub.exchange(self.rank, t.clone())
        return [got[r] for r in range(self.world)]

    def all_to_all(self, parts):
        got = self.hub.exchange(self.rank, [p.clone() for p in parts])
        return [got[r][self.rank] for r in range(self.world)]

    def broadcast(self, t, src=0):
        got = self.hub.exchange(self.rank, t.clone() if self.rank == src else None)
        return got[src]

    def all_reduce_scalar(self, v, op="max"):
        got = self.hub.exchange(self.rank, float(v))
        vals = [got[r] for r in range(self.world)]
        return {"max": max, "min": min, "sum": sum}[op](vals)

    def barrier(self):
        self.hub.exchange(self.rank, None)

    def host_signal(self, key, value="1"):
        self.hub.signal(key, value)

    def host_wait(self, key, timeout_s=60.0):
        return self.hub.wait(key, timeout_s)


# ---------------------------------------------------------------------------- process group
class GroupComm(Comm):
    """``torch.distributed`` backend: NCCL for CUDA tensors, gloo for CPU tensors (chosen by the group's
    backend, never by catching errors)."""

    def __init__(self, group=None, store=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = dist.get_backend(group)
        self.store = store

    def _dev(self, t):
        return t

    def all_gather(self, t):
        dist = self.dist
        n = torch.tensor([t.shape[0]], device=t.device, dtype=torch.int64)
        ns = [torch.zeros_like(n) for _ in range(self.world)]
        dist.all_gather(ns, n, group=self.group)
        sizes = [int(x.item()) for x in ns]
        mx = max(sizes)
        pad = t
        if t.shape[0] < mx:
            pad = torch.cat([t, t.new_zeros((mx - t.shape[0],) + tuple(t.shape[1:]))], 0)
        outs = [torch.empty_like(pad) for _ in range(self.world)]
        dist.all_gather(outs, pad.contiguous(), group=self.group)
        return [o[:s] for o, s in zip(outs, sizes)]

    def all_to_all(self, parts):
        dist = self.dist
        shapes = self._exchange_shapes(parts)
        outs = [torch.empty(shapes[q], dtype=parts[0].dtype, device=parts[0].device) for q in range(self.world)]
        if self.backend == "nccl":
            dist.all_to_all(outs, [p.contiguous() for p in parts], group=self.group)
        else:
            # gloo has no all_to_all: pairwise exchange in a fixed order
            reqs = []
            for q in range(self.world):
                if q == self.rank:
                    outs[q].copy_(parts[q])
                else:
                    reqs.append(dist.isend(parts[q].contiguous(), q, group=self.group))
                    reqs.append(dist.irecv(outs[q], q, group=self.group))
            for r in reqs:
                r.wait()
        return outs

    def _exchange_shapes(self, parts):
        dist = self.dist
        nd = parts[0].dim()
        mine = torch.tensor([list(p.shape) for p in parts], dtype=torch.int64, device=parts[0].device)   # [P, nd]
        allv = [torch.zeros_like(mine) for _ in range(self.world)]
        dist.all_gather(allv, mine, group=self.group)
        return [tuple(int(x) for x in allv[q][self.rank].tolist()) for q in range(self.world)]

    def broadcast(self, t, src=0):
        self.dist.broadcast(t, src, group=self.group)
        return t

    def all_reduce_scalar(self, v, op="max"):
        dist = self.dist
        dev = "cuda" if self.backend == "nccl" else "cpu"
        x = torch.tensor([float(v)], dtype=torch.float64, device=dev)
        dist.all_reduce(x, {"max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN, "sum": dist.ReduceOp.SUM}[op],
                        group=self.group)
        return float(x.item())

    def barrier(self):
        self.dist.barrier(group=self.group)

    def host_signal(self, key, value="1"):
        if self.store is None:
            raise CommAborted("no store for host signalling")
        self.store.set(key, value)

    def host_wait(self, key, timeout_s=60.0):
        if self.store is None:
            raise CommAborted("no store for host signalling")
        import datetime
        try:
            self.store.wait([key], datetime.timedelta(seconds=timeout_s))
        except Exception as e:  # noqa: BLE001
            raise CommAborted(f"host_wait({key}) timed out after {timeout_s}s: {e}") from e
        return self.store.get(key).decode()
