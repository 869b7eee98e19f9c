"""Cold start: build a model without the random initialisation a checkpoint load overwrites, and read the
checkpoint without a second copy.

:func:`no_init` makes the ``torch.nn.init`` fillers no-ops while modules construct (parameters allocated, not
filled; it counts the skipped calls); :func:`meta_init` constructs on the ``meta`` device and
:func:`materialize` assigns a state dict into it; :func:`load_total` is ``load_state_dict`` plus the totality
proof (every parameter and persistent buffer came from the checkpoint - a missing key refuses by name, since an
uninitialised tensor would otherwise survive); :func:`mmap_state_dict` memory-maps a checkpoint;
:func:`state_digest` is the sha256 over (name, dtype, shape, bytes) that shows two loads are equal.
Reference: common/opt_core/opt_core/host/coldstart.py, host_cache/fast_init.py.
"""
from __future__ import annotations

import contextlib
import hashlib
from typing import Dict, Iterable, List, Mapping

import torch
import torch.nn as nn


class PartialLoad(RuntimeError):
    pass


_FILLERS = ["uniform_", "normal_", "trunc_normal_", "constant_", "ones_", "zeros_", "eye_", "dirac_",
            "xavier_uniform_", "xavier_normal_", "kaiming_uniform_", "kaiming_normal_", "orthogonal_", "sparse_"]


class _Counter:
    n = 0


@contextlib.contextmanager
def no_init():
    """``with no_init() as c: model = Model(cfg)`` - init fillers write nothing inside; ``c.n`` = calls skipped."""
    c = _Counter()
    saved = {}

    def skip(t, *a, **k):
        c.n += 1
        return t

    for name in _FILLERS:
        if hasattr(nn.init, name):
            saved[name] = getattr(nn.init, name)
            setattr(nn.init, name, skip)
    try:
        yield c
    finally:
        for name, fn in saved.items():
            setattr(nn.init, name, fn)


@contextlib.contextmanager
def meta_init():
    with torch.device("meta"):
        yield


def _expected_keys(module: nn.Module) -> List[str]:
    return list(module.state_dict().keys())


def load_total(module: nn.Module, state: Mapping[str, torch.Tensor], allow_unexpected: Iterable[str] = ()) -> int:
    """``load_state_dict(strict=False)`` + the proof that nothing was left as constructed."""
    res = module.load_state_dict(state, strict=False)
    if res.missing_keys:
        raise PartialLoad(f"checkpoint lacks {len(res.missing_keys)} tensors, first: {res.missing_keys[0]}")
    extra = [k for k in res.unexpected_keys if k not in set(allow_unexpected)]
    if extra:
        raise PartialLoad(f"checkpoint has {len(extra)} tensors the model does not, first: {extra[0]}")
    return len(_expected_keys(module))


def materialize(module: nn.Module, state: Mapping[str, torch.Tensor]) -> int:
    """Assign ``state`` into a meta-constructed module (no copy of the weights), then the totality proof."""
    res = module.load_state_dict(state, strict=False, assign=True)
    if res.missing_keys:
        raise PartialLoad(f"checkpoint lacks {len(res.missing_keys)} tensors, first: {res.missing_keys[0]}")
    left = [n for n, p in list(module.named_parameters()) + list(module.named_buffers()) if p.is_meta]
    if left:
        raise PartialLoad(f"{len(left)} tensors still on the meta device, first: {left[0]}")
    return len(_expected_keys(module))


def mmap_state_dict(path: str) -> Dict[str, torch.Tensor]:
    return torch.load(path, mmap=True, map_location="cpu", weights_only=True)


def state_digest(module_or_state) -> str:
    state = module_or_state.state_dict() if isinstance(module_or_state, nn.Module) else module_or_state
    h = hashlib.sha256()
    for name in sorted(state):
        t = state[name].detach().cpu().contiguous()
        h.update(name.encode() + str(t.dtype).encode() + str(tuple(t.shape)).encode())
        h.update(t.view(torch.uint8).numpy().tobytes() if t.numel() else b"")
    return h.hexdigest()
