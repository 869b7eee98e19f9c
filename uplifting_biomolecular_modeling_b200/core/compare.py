"""Compare output trees: sha256 of every file, and numeric comparison of tensors within a tolerance.
``exact`` runs are held to equal digests, ``fast`` runs to a stated relative tolerance.
Reference: common/opt_core/opt_core/compare.py:24."""
from __future__ import annotations

import os
from typing import Dict, Mapping, Tuple

from .gates import sha256_file


def tree_digests(root: str) -> Dict[str, str]:
    out = {}
    for d, _, files in os.walk(root):
        for f in sorted(files):
            p = os.path.join(d, f)
            out[os.path.relpath(p, root)] = sha256_file(p)
    return out


def diff_trees(a: str, b: str, ignore=("opt_manifest.json",)) -> Dict[str, str]:
    da, db = tree_digests(a), tree_digests(b)
    out = {}
    for k in sorted(set(da) | set(db)):
        if os.path.basename(k) in ignore:
            continue
        if k not in da:
            out[k] = "only_in_b"
        elif k not in db:
            out[k] = "only_in_a"
        elif da[k] != db[k]:
            out[k] = "differs"
    return out


def tensors_close(a: Mapping, b: Mapping, rtol: float = 1e-3) -> Tuple[bool, Dict[str, float]]:
    """Max relative error per key (|a-b|_max / |b|_max)."""
    import torch
    errs = {}
    ok = True
    for k in a:
        if k not in b:
            ok = False
            errs[k] = float("inf")
            continue
        x, y = torch.as_tensor(a[k]).float(), torch.as_tensor(b[k]).float()
        e = ((x - y).abs().max() / y.abs().max().clamp(min=1e-12)).item() if x.numel() else 0.0
        errs[k] = e
        ok = ok and e <= rtol
    return ok, errs
