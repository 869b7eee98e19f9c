"""Attention-backend pin and memory budgets of the sequence-model kits.

``pinned_backend(name)`` is a context manager that restricts the library's scaled-dot-product attention to one
named backend for the duration of a forward (an ``exact`` mode must not let the dispatcher pick a different
kernel from one batch shape to the next); unknown names are refused.  ``tokens_within(free_bytes, ...)`` turns a
free-memory figure into a token ceiling for the batch planner.  Reference: common/opt_core/opt_core/seq/*.py
(attention-backend pin, mem budgets).
"""
from __future__ import annotations

import contextlib
from typing import Optional

import torch

BACKENDS = ("math", "flash", "efficient", "cudnn")


def _enum(name: str):
    from torch.nn.attention import SDPBackend
    return {"math": SDPBackend.MATH, "flash": SDPBackend.FLASH_ATTENTION, "efficient": SDPBackend.EFFICIENT_ATTENTION,
            "cudnn": SDPBackend.CUDNN_ATTENTION}[name]


@contextlib.contextmanager
def pinned_backend(name: str):
    if name not in BACKENDS:
        raise ValueError(f"attention backend {name!r} not in {BACKENDS}")
    from torch.nn.attention import sdpa_kernel
    with sdpa_kernel(_enum(name)):
        yield name


def tokens_within(free_bytes: int, d_model: int, layers: int, bytes_per_element: int = 2, live_per_layer: float = 6.0,
                  reserve: float = 0.15, ceiling: Optional[int] = None) -> int:
    """Largest token count whose activations fit: ``live_per_layer`` row-sized tensors are alive inside a layer,
    plus one residual row per layer boundary; ``reserve`` of the free memory is left to the allocator."""
    usable = int(free_bytes * (1.0 - reserve))
    per_token = int(d_model * bytes_per_element * (live_per_layer + 1))
    n = max(0, usable // max(1, per_token))
    return n if ceiling is None else min(n, ceiling)
