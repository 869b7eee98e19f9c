"""Digests of things that come from outside the repository: weight files and state dicts.

``weight_digest`` hashes tensor names, dtypes, shapes and bytes in sorted name order, so two checkpoints with
the same parameters have the same digest whatever container they came in; ``file_digest`` streams a file;
``check`` refuses by name when a digest differs from the pin.  Reference: common/opt_core/opt_core/extern.py.
"""
from __future__ import annotations

import hashlib
from typing import Mapping, Optional


class DigestMismatch(RuntimeError):
    pass


def file_digest(path: str, chunk: int = 1 << 22) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def weight_digest(state: Mapping[str, "torch.Tensor"]) -> str:
    import torch  # noqa: PLC0415 - the contract runtime stays importable without the tensor library
    h = hashlib.sha256()
    for name in sorted(state):
        t = state[name].detach().cpu().contiguous()
        h.update(name.encode())
        h.update(str(t.dtype).encode())
        h.update(str(tuple(t.shape)).encode())
        h.update(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    return h.hexdigest()


def check(what: str, got: str, pinned: Optional[str]) -> None:
    if pinned is not None and got != pinned:
        raise DigestMismatch(f"{what}: digest {got[:16]}... differs from the pinned {pinned[:16]}...")
