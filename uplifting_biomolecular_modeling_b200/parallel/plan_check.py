"""Host-side checks of peer-memory exchanges before any kernel is launched.

* :func:`check_exchange_plan` - every rank lists the transfers it will issue (``Transfer(kind, peer, tag,
  nbytes)`` with kind ``"put"`` / ``"get"`` for one-sided peer stores / loads and ``"send"`` / ``"recv"`` for
  two-sided ones); the check refuses, by name, plans where a send has no matching receive (or the sizes
  differ), where two ranks order their two-sided transfers with each other differently (a deadlock with blocking
  transports), where a one-sided transfer targets a rank outside the group or exceeds the registered size of its
  target buffer, or where two puts of one step overlap in the same target range.
* :class:`CanaryBuffer` - a peer-visible buffer with guard words before and after its payload;
  :meth:`CanaryBuffer.check` names the side that was overwritten.

Reference: the pre-post matching of every p2p send / recv set (common/opt_core/opt_core/mem/rowpair/dist.py:455,
``ROWPAIR_P2P_CHECK=1``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Mapping, Optional, Sequence, Tuple

import torch


class PlanMismatch(RuntimeError):
    pass


@dataclass(frozen=True)
class Transfer:
    kind: str                 # send | recv | put | get
    peer: int
    tag: str
    nbytes: int
    offset: int = 0           # byte offset inside the target buffer (one-sided transfers)


def check_exchange_plan(plans: Mapping[int, Sequence[Transfer]],
                        buffer_bytes: Optional[Mapping[Tuple[int, str], int]] = None) -> int:
    """``plans[rank]`` is the ordered list of transfers that rank issues in one step.  ``buffer_bytes[(rank, tag)]``
    is the registered size of rank's buffer ``tag`` (checked for one-sided transfers when given).  Returns the
    number of matched transfers; raises :class:`PlanMismatch` naming the first problem."""
    world = sorted(plans)
    ranks = set(world)
    matched = 0
    for r in world:
        for t in plans[r]:
            if t.kind not in ("send", "recv", "put", "get"):
                raise PlanMismatch(f"rank {r}: unknown transfer kind {t.kind!r}")
            if t.peer not in ranks:
                raise PlanMismatch(f"rank {r}: {t.kind} {t.tag!r} names rank {t.peer}, outside the group {world}")
            if t.nbytes < 0 or t.offset < 0:
                raise PlanMismatch(f"rank {r}: {t.kind} {t.tag!r} has a negative size or offset")
    # two-sided: per ordered pair, the sequence of (tag, nbytes) sent must equal the sequence received
    for a in world:
        for b in world:
            if a == b:
                continue
            sends = [(t.tag, t.nbytes) for t in plans[a] if t.kind == "send" and t.peer == b]
            recvs = [(t.tag, t.nbytes) for t in plans[b] if t.kind == "recv" and t.peer == a]
            if sorted(sends) != sorted(recvs):
                missing = [s for s in sends if s not in recvs] or [x for x in recvs if x not in sends]
                raise PlanMismatch(f"ranks {a} -> {b}: sends and receives do not pair up (first unmatched: {missing[0]})")
            if sends != recvs:
                raise PlanMismatch(f"ranks {a} -> {b}: transfers are posted in different orders "
                                   f"({[s[0] for s in sends]} vs {[x[0] for x in recvs]})")
            matched += len(sends)
    # pairwise progress: if a's first two-sided transfer with b is a blocking send while b's first with a is also a
    # send, neither receive is posted
    for a in world:
        for b in world:
            if a >= b:
                continue
            fa = next((t.kind for t in plans[a] if t.peer == b and t.kind in ("send", "recv")), None)
            fb = next((t.kind for t in plans[b] if t.peer == a and t.kind in ("send", "recv")), None)
            if fa == "recv" and fb == "recv":
                raise PlanMismatch(f"ranks {a} and {b} both start by receiving from each other")
    # one-sided: bounds and overlapping puts
    writes: Dict[Tuple[int, str], List[Tuple[int, int, int]]] = {}
    for r in world:
        for t in plans[r]:
            if t.kind not in ("put", "get"):
                continue
            size = None if buffer_bytes is None else buffer_bytes.get((t.peer, t.tag))
            if buffer_bytes is not None and size is None:
                raise PlanMismatch(f"rank {r}: {t.kind} {t.tag!r} targets a buffer that rank {t.peer} did not register")
            if size is not None and t.offset + t.nbytes > size:
                raise PlanMismatch(f"rank {r}: {t.kind} {t.tag!r} [{t.offset}, {t.offset + t.nbytes}) exceeds the "
                                   f"{size} bytes registered on rank {t.peer}")
            if t.kind == "put":
                writes.setdefault((t.peer, t.tag), []).append((t.offset, t.offset + t.nbytes, r))
            matched += 1
    for (peer, tag), spans in writes.items():
        spans.sort()
        for (s0, e0, r0), (s1, e1, r1) in zip(spans, spans[1:]):
            if s1 < e0:
                raise PlanMismatch(f"puts of ranks {r0} and {r1} overlap in buffer {tag!r} of rank {peer} "
                                   f"([{s0}, {e0}) and [{s1}, {e1}))")
    return matched


def row_gather_plan(world: int, rows_per_rank: Sequence[int], row_bytes: int, tag: str = "rows") -> Dict[int, List[Transfer]]:
    """The plan of the gather-once exchange: every rank pulls every other rank's row block into its gathered buffer
    (one ``get`` per remote block, at the block's row offset)."""
    return {r: [Transfer("get", q, tag, rows_per_rank[q] * row_bytes, 0) for q in range(world) if q != r]
            for r in range(world)}


def reduce_scatter_plan(world: int, rows_per_rank: Sequence[int], row_bytes: int, tag: str = "slots") -> Dict[int, List[Transfer]]:
    """The plan of the GEMM epilogue's reduce-scatter: rank r stores its partial rows of owner q into slot r of q's
    slot buffer."""
    return {r: [Transfer("put", q, tag, rows_per_rank[q] * row_bytes, r * rows_per_rank[q] * row_bytes)
                for q in range(world)] for r in range(world)}


CANARY = 0x5AFEC0DE


class CanaryBuffer:
    """``payload`` is a view into an allocation with ``guard`` int32 words of a fixed pattern on either side."""

    def __init__(self, nbytes: int, device="cpu", guard: int = 16):
        self.guard = guard
        words = (nbytes + 3) // 4
        self.raw = torch.empty(words + 2 * guard, dtype=torch.int32, device=device)
        self.raw[:guard] = CANARY
        self.raw[guard + words:] = CANARY
        self.payload = self.raw[guard:guard + words]

    def check(self, what: str = "buffer") -> None:
        g = self.guard
        head_ok = bool((self.raw[:g] == CANARY).all())
        tail_ok = bool((self.raw[g + self.payload.numel():] == CANARY).all())
        if not head_ok or not tail_ok:
            side = "before" if not head_ok else "after"
            raise PlanMismatch(f"{what}: guard words {side} the payload were overwritten")
