"""Allocator policy of ``big``: expandable segments (verified by reading the allocator configuration back),
cache release between stages.  Reference: common/opt_core/opt_core/mem/allocator.py:177,224."""
from __future__ import annotations

import os
from typing import Optional

from .registry import Ctx, Refusal, register

ENV = "PYTORCH_CUDA_ALLOC_CONF"


def want_expandable(environ: Optional[dict] = None) -> bool:
    """Set ``expandable_segments:True`` in the allocator configuration (before CUDA starts)."""
    env = os.environ if environ is None else environ
    cur = env.get(ENV, "")
    if "expandable_segments" in cur:
        return "expandable_segments:True" in cur
    env[ENV] = (cur + "," if cur else "") + "expandable_segments:True"
    return True


def verify_expandable() -> Optional[bool]:
    """Read the live allocator setting back; None when it cannot be read."""
    try:
        import torch
        if not torch.cuda.is_available():
            return None
        snap = torch.cuda.memory._snapshot()
        cfg = snap.get("allocator_settings", {})
        return bool(cfg.get("expandable_segments"))
    except Exception:  # noqa: BLE001
        return None


def cache_release() -> int:
    """Return cached blocks to the driver; returns the bytes still reserved."""
    import torch
    if not torch.cuda.is_available():
        return 0
    torch.cuda.empty_cache()
    return int(torch.cuda.memory_reserved())


@register("expandable_segments", label="bitwise", droppable=True)
def _lever_expandable(ctx: Ctx):
    ok = want_expandable(ctx.settings.get("environ"))
    live = verify_expandable()
    if live is False:
        raise Refusal("allocator_already_initialised")
    return {"requested": ok, "verified": live}


@register("cache_release", label="bitwise", droppable=True)
def _lever_cache_release(ctx: Ctx):
    return {"reserved_after": cache_release()}
