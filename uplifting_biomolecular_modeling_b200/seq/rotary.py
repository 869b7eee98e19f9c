"""Resident rotary tables: cos / sin computed once per (head_dim, base, device) and extended on demand, instead
of being rebuilt in every attention call."""
from __future__ import annotations

from typing import Dict, Tuple

import torch


class RotaryTable:
    _tables: Dict[Tuple, "RotaryTable"] = {}

    def __init__(self, head_dim: int, base: float = 10000.0, device="cpu"):
        self.head_dim, self.base, self.device = head_dim, base, torch.device(device)
        self.cos = torch.empty((0, head_dim // 2), device=self.device)
        self.sin = torch.empty((0, head_dim // 2), device=self.device)
        self.builds = 0

    @classmethod
    def get(cls, head_dim: int, base: float = 10000.0, device="cpu") -> "RotaryTable":
        key = (head_dim, float(base), str(torch.device(device)))
        if key not in cls._tables:
            cls._tables[key] = cls(head_dim, base, device)
        return cls._tables[key]

    def upto(self, length: int):
        """cos, sin of positions [0, length): [length, head_dim / 2] fp32."""
        if length > self.cos.shape[0]:
            n = max(length, 2 * self.cos.shape[0], 256)
            inv = 1.0 / (self.base ** (torch.arange(0, self.head_dim, 2, device=self.device, dtype=torch.float32)
                                       / self.head_dim))
            ang = torch.arange(n, device=self.device, dtype=torch.float32).unsqueeze(-1) * inv
            self.cos, self.sin = ang.cos(), ang.sin()
            self.builds += 1
        return self.cos[:length], self.sin[:length]

    def apply(self, x: torch.Tensor, pos: torch.Tensor) -> torch.Tensor:
        """Interleaved-pair rotary of x [..., L, heads, head_dim] at integer positions pos [L] (a device tensor:
        the lookup is a gather, no host value)."""
        cos, sin = self.upto(int(self.cos.shape[0]) if pos.is_cuda and self.cos.shape[0] else int(pos.max()) + 1)
        c, s = cos[pos][:, None, :], sin[pos][:, None, :]
        x1, x2 = x.float()[..., 0::2], x.float()[..., 1::2]
        return torch.stack([x1 * c - x2 * s, x1 * s + x2 * c], -1).flatten(-2).to(x.dtype)
