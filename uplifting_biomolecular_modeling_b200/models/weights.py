"""Loading upstream checkpoints unchanged.

The model classes use upstream parameter names, so a checkpoint loads by name after stripping the wrapper
prefixes the upstream trainers add (Lightning ``state_dict`` with ``model.`` / ``module.`` prefixes, EMA
copies under ``ema.`` ...).  ``load_checkpoint`` reports what matched; a checkpoint that matches nothing is
an error, missing or unexpected keys are returned for the caller's manifest.  File digests can be held to a
pin (``expected_sha256``) before anything is unpickled.
Reference: boltz2/stock/PINS.json ``weights``, common/opt_core/opt_core/extern.py (weight digests),
host/coldstart.py (meta-device init + mmap load).
"""
from __future__ import annotations

from typing import Dict, Iterable, Optional, Tuple

import torch

from ..core.gates import sha256_file

PREFIXES = ("model.", "module.", "structure_module.score_model.module.", "_orig_mod.", "ema.", "ema_model.")


def strip_prefixes(state: Dict[str, torch.Tensor], prefixes: Iterable[str] = PREFIXES) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state.items():
        changed = True
        while changed:
            changed = False
            for p in prefixes:
                if k.startswith(p):
                    k = k[len(p):]
                    changed = True
        out[k] = v
    return out


def read_state(path: str, expected_sha256: Optional[str] = None) -> Dict[str, torch.Tensor]:
    if expected_sha256 is not None and sha256_file(path) != expected_sha256:
        raise ValueError(f"checkpoint digest mismatch: {path}")
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file  # type: ignore
        return load_file(path)
    obj = torch.load(path, map_location="cpu", mmap=True, weights_only=False)
    if isinstance(obj, dict):
        for key in ("state_dict", "model", "model_state_dict", "ema"):
            if key in obj and isinstance(obj[key], dict):
                return obj[key]
    return obj


def load_checkpoint(model: torch.nn.Module, path: str, expected_sha256: Optional[str] = None,
                    strict: bool = False) -> Tuple[int, list, list]:
    """Returns (matched, missing, unexpected)."""
    state = strip_prefixes(read_state(path, expected_sha256))
    own = model.state_dict()
    matched = {k: v for k, v in state.items() if k in own and tuple(own[k].shape) == tuple(v.shape)}
    if not matched:
        raise ValueError(f"{path}: no parameter of the checkpoint matches the model by name and shape")
    missing = sorted(k for k in own if k not in matched)
    unexpected = sorted(k for k in state if k not in matched)
    if strict and (missing or unexpected):
        raise ValueError(f"{path}: {len(missing)} missing / {len(unexpected)} unexpected parameters")
    model.load_state_dict({k: v.to(own[k].dtype) for k, v in matched.items()}, strict=False)
    for m in model.modules():                      # packed (folded) weights are rebuilt from the new parameters
        if hasattr(m, "_packed"):
            m._packed = None
    return len(matched), missing, unexpected


def meta_init(build_fn, *args, **kw):
    """Build a model without running random initialisation (parameters on the meta device); the caller
    materialises them with ``load_checkpoint`` after ``to_empty``."""
    with torch.device("meta"):
        return build_fn(*args, **kw)
