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

from dataclasses import dataclass, field
from typing import Dict, Iterable, List, Optional

import torch

from ..core.gates import sha256_file

PREFIXES = ("model.", "module.", "structure_module.score_model.module.", "_orig_mod.", "ema.", "ema_model.")


EMA_PREFIXES = ("ema.", "ema_model.")


class KeyCollision(ValueError):
    """Two checkpoint entries map to one parameter name after the wrapper prefixes are stripped."""


def _strip(k: str, prefixes) -> str:
    changed = True
    while changed:
        changed = False
        for p in prefixes:
            if k.startswith(p):
                k = k[len(p):]
                changed = True
    return k


def strip_prefixes(state: Dict[str, torch.Tensor], prefixes: Iterable[str] = PREFIXES,
                   ema: Optional[bool] = None) -> Dict[str, torch.Tensor]:
    """Parameter names without the trainers' wrapper prefixes.  A checkpoint that carries both the raw and the
    averaged (``ema.``) copy of a parameter maps two entries to one name: ``ema=True`` / ``ema=False`` says which
    copy to take; with ``ema=None`` such a checkpoint raises :class:`KeyCollision` instead of letting the later
    entry win."""
    prefixes = tuple(prefixes)
    groups: Dict[str, list] = {}
    for k, v in state.items():
        groups.setdefault(_strip(k, prefixes), []).append((k, k.startswith(EMA_PREFIXES), v))
    out: Dict[str, torch.Tensor] = {}
    for name, entries in groups.items():
        if len(entries) > 1:
            keys = ", ".join(repr(e[0]) for e in entries)
            if ema is None:
                raise KeyCollision(f"checkpoint entries {keys} all map to {name!r} (pass ema=True or ema=False)")
            entries = [e for e in entries if e[1] == ema]
            if len(entries) != 1:
                raise KeyCollision(f"checkpoint entries {keys} map to {name!r}; ema={ema} does not single one out")
        out[name] = entries[0][2]
    return out


def read_state(path: str, expected_sha256: Optional[str] = None) -> Dict[str, torch.Tensor]:
    if expected_sha256 is not None and sha256_file(path) != expected_sha256:
        raise ValueError(f"checkpoint digest mismatch: {path}")
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file  # type: ignore
        return load_file(path)
    try:
        obj = torch.load(path, map_location="cpu", mmap=True, weights_only=True)
    except Exception:  # noqa: BLE001 - a pickle with non-tensor objects (Lightning hyper-parameters, ...)
        if expected_sha256 is None:
            raise ValueError(f"{path}: not loadable as tensors only; unpickling arbitrary objects needs a pinned "
                             f"sha256 of the file (expected_sha256)") from None
        obj = torch.load(path, map_location="cpu", mmap=True, weights_only=False)
    if isinstance(obj, dict):
        for key in ("state_dict", "model", "model_state_dict", "ema"):
            if key in obj and isinstance(obj[key], dict):
                return obj[key]
    return obj


@dataclass
class LoadReport:
    matched: int = 0
    missing: List[str] = field(default_factory=list)          # parameters of the model the checkpoint lacks
    unexpected: List[str] = field(default_factory=list)       # checkpoint entries the model has no parameter for
    shape_mismatch: List[str] = field(default_factory=list)   # same name, other shape: "name: ckpt (..) model (..)"

    @property
    def complete(self) -> bool:
        return not (self.missing or self.unexpected or self.shape_mismatch)

    def __iter__(self):                                        # (matched, missing, unexpected) for older callers
        return iter((self.matched, self.missing, self.unexpected))


def load_checkpoint(model: torch.nn.Module, path: str, expected_sha256: Optional[str] = None,
                    strict: bool = True, ema: Optional[bool] = None, mapper=None, dry_run: bool = False) -> LoadReport:
    """Load by name after prefix stripping (and after ``mapper``, a function state -> state that translates an
    upstream's parameter names into this package's: :mod:`models.mappers`).  ``strict`` (the default): every parameter of the model must be in the
    checkpoint with its shape and the checkpoint may hold nothing else, otherwise ``ValueError`` - a run on partly
    random weights is never silent.  ``strict=False`` loads what matches and reports the rest.  ``dry_run`` checks
    names and shapes (and raises as above) without writing a parameter - a launcher holds a checkpoint against a
    model built on the meta device before it starts rank processes."""
    state = strip_prefixes(read_state(path, expected_sha256), ema=ema)
    if mapper is not None:
        state = mapper(state)
    own = model.state_dict()
    rep = LoadReport()
    matched = {}
    for k, v in state.items():
        if k not in own:
            rep.unexpected.append(k)
        elif tuple(own[k].shape) != tuple(v.shape):
            rep.shape_mismatch.append(f"{k}: checkpoint {tuple(v.shape)} model {tuple(own[k].shape)}")
        else:
            matched[k] = v
    rep.missing = sorted(k for k in own if k not in matched and not any(s_.startswith(k + ":") for s_ in rep.shape_mismatch))
    rep.unexpected.sort()
    rep.matched = len(matched)
    if not matched:
        raise ValueError(f"{path}: no parameter of the checkpoint matches the model by name and shape")
    if strict and not rep.complete:
        raise ValueError(f"{path}: {len(rep.missing)} missing / {len(rep.unexpected)} unexpected / "
                         f"{len(rep.shape_mismatch)} shape-mismatched parameters (first: "
                         f"{(rep.missing + rep.unexpected + rep.shape_mismatch)[0]})")
    if dry_run:                                    # names and shapes only: the model may live on the meta device
        return rep
    model.load_state_dict({k: v.to(own[k].dtype) for k, v in matched.items()}, strict=False)
    for m in model.modules():                      # packed (folded) weights are rebuilt from the new parameters
        if hasattr(m, "_packed"):
            m._packed = None
    return rep


def meta_init(build_fn, *args, **kw):
    """Build a model without running random initialisation (parameters on the meta device); the caller
    materialises them with ``load_checkpoint`` after ``to_empty``."""
    with torch.device("meta"):
        return build_fn(*args, **kw)
