"""Memory mode (``big``): levers that lower the peak device memory of one prediction on one GPU -
row-chunked pair operations, early release, host parking with a streamed device window, allocator policy,
sample chunking - and the record of what was applied.  The multi-GPU form of ``big`` lives in ``parallel``."""
from .registry import Ctx, Lever, Refusal, apply, register, registered  # noqa: F401
