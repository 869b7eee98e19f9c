"""Variable-length batches without a host synchronisation: cumulative sequence lengths computed on the device from
the mask, never through ``.item()`` / ``.tolist()``."""
from __future__ import annotations

import torch


def cu_seqlens(mask: torch.Tensor) -> torch.Tensor:
    """mask: [B, L] (1 = token) -> int32 [B + 1] cumulative lengths, on mask's device, no host value read."""
    lens = mask.to(torch.int32).sum(1)
    return torch.nn.functional.pad(torch.cumsum(lens, 0, dtype=torch.int32), (1, 0))


def pad_to_multiple(x: torch.Tensor, multiple: int, dim: int = 1, value: float = 0.0) -> torch.Tensor:
    n = x.shape[dim]
    extra = (-n) % multiple
    if not extra:
        return x
    pad = [0, 0] * (x.dim() - 1 - dim) + [0, extra]
    return torch.nn.functional.pad(x, pad, value=value)
