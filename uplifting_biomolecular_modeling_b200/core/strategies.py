"""Catalogue of strategy ids used on LEVER lines (``F<k>.<name>`` families, ``LOCAL.<kit>.<name>``).
Reference: common/opt_core/opt_core/strategies.py:29."""
from __future__ import annotations

FAMILIES = {
    "F1.kernel_fusion": "several statements served by one kernel (same math, fewer passes over HBM)",
    "F2.graph_capture": "launch-bound loops replayed from CUDA graphs",
    "F3.hoisting": "step- or layer-invariant work computed once",
    "F4.precision": "documented reduced-precision arithmetic (bf16 pair stack, TF32, e4m3 input projections)",
    "F5.memory": "chunking, early release, offload, allocator policy",
    "F6.host_overlap": "prefetch, background writers, resident workers",
    "F7.tensor_parallel": "one prediction sharded over the GPUs of a host",
    "F8.weights": "one-time weight transforms (folding LayerNorm, packing, casting)",
}


def is_known(sid: str) -> bool:
    return sid in FAMILIES or sid.startswith("LOCAL.")


def local(kit: str, name: str) -> str:
    return f"LOCAL.{kit}.{name}"
