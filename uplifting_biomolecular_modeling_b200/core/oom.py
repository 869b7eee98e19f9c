"""One classifier for out-of-memory conditions (exception object or log text), so that every caller
agrees on what counts as OOM.  Reference: common/opt_core/opt_core/oom.py:47,59."""
from __future__ import annotations

import re

_PATTERNS = (r"CUDA out of memory", r"out of memory", r"CUDA_ERROR_OUT_OF_MEMORY", r"cudaErrorMemoryAllocation",
             r"RESOURCE_EXHAUSTED", r"OutOfMemoryError", r"NCCL.*unhandled cuda error.*memory",
             r"std::bad_alloc", r"Cannot allocate memory")
_RX = re.compile("|".join(_PATTERNS), re.IGNORECASE)


def is_oom_text(text: str) -> bool:
    return bool(text) and bool(_RX.search(text))


def is_oom(exc: BaseException) -> bool:
    name = type(exc).__name__
    if name in ("OutOfMemoryError", "MemoryError"):
        return True
    return is_oom_text(str(exc))
