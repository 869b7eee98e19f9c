"""Determinism recipe and numerics policy.

``Recipe`` names what a deterministic run pins (seeds, deterministic algorithms, cuDNN benchmark
off, TF32 policy, the cuBLAS workspace variable); ``apply_env`` sets the environment part before
CUDA starts, ``apply_switches`` the in-process part.  ``numerics_signature`` is a short string of
the settings that change floating-point results, stored in manifests and checkpoints so that a resume
under a different signature is refused.  ``segment_sum`` is the deterministic replacement of an
atomic scatter-add.  Reference: common/opt_core/opt_core/det.py:18, precision/policy.py:64,276,353,
precision/recipe.py:72,129, precision/det_scatter.py:104,175.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, asdict
from typing import Mapping, Optional


@dataclass(frozen=True)
class Recipe:
    seed: int = 0
    deterministic_algorithms: bool = True
    cudnn_benchmark: bool = False
    allow_tf32: bool = False
    matmul_precision: str = "highest"          # highest | high | medium
    cublas_workspace: str = ":4096:8"
    python_hash_seed: str = "0"


@dataclass(frozen=True)
class Policy:
    """Numerics of a mode: compute dtype of the pair stack, TF32, autocast."""
    compute_dtype: str = "bf16"
    allow_tf32: bool = False
    autocast: bool = False
    matmul_precision: str = "highest"


def apply_env(recipe: Recipe, environ: Optional[dict] = None) -> dict:
    env = os.environ if environ is None else environ
    env.setdefault("CUBLAS_WORKSPACE_CONFIG", recipe.cublas_workspace)
    env.setdefault("PYTHONHASHSEED", recipe.python_hash_seed)
    return env


def apply_switches(recipe: Recipe) -> dict:
    """Seed and switch torch; returns what was set (also usable without CUDA)."""
    import torch
    torch.manual_seed(recipe.seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(recipe.seed)
    torch.use_deterministic_algorithms(recipe.deterministic_algorithms, warn_only=True)
    torch.backends.cudnn.benchmark = recipe.cudnn_benchmark
    torch.backends.cuda.matmul.allow_tf32 = recipe.allow_tf32
    torch.backends.cudnn.allow_tf32 = recipe.allow_tf32
    torch.set_float32_matmul_precision(recipe.matmul_precision)
    return asdict(recipe)


def numerics_signature(policy: Policy, extra: Optional[Mapping] = None) -> str:
    parts = [f"dtype={policy.compute_dtype}", f"tf32={int(policy.allow_tf32)}", f"autocast={int(policy.autocast)}",
             f"matmul={policy.matmul_precision}"]
    try:
        import torch
        parts.append(f"torch={torch.__version__.split('+')[0]}")
    except Exception:  # noqa: BLE001
        pass
    for k in sorted(extra or {}):
        parts.append(f"{k}={extra[k]}")
    return ";".join(parts)


class NumericsGuard:
    """Context manager that applies a policy and restores the previous switches."""

    def __init__(self, policy: Policy):
        self.policy = policy
        self._old = None

    def __enter__(self):
        import torch
        self._old = (torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32,
                     torch.get_float32_matmul_precision())
        torch.backends.cuda.matmul.allow_tf32 = self.policy.allow_tf32
        torch.backends.cudnn.allow_tf32 = self.policy.allow_tf32
        torch.set_float32_matmul_precision(self.policy.matmul_precision)
        return self

    def __exit__(self, *exc):
        import torch
        torch.backends.cuda.matmul.allow_tf32, torch.backends.cudnn.allow_tf32 = self._old[0], self._old[1]
        torch.set_float32_matmul_precision(self._old[2])
        return False


def segment_sum(values, segment_ids, num_segments: int):
    """Deterministic sum of rows per segment (sorted by segment, summed by a cumulative-sum difference in
    float64), replacing ``index_add_`` whose atomics make the order of additions vary run to run."""
    import torch
    order = torch.argsort(segment_ids, stable=True)
    v = values[order].to(torch.float64)
    ids = segment_ids[order]
    cs = torch.cumsum(v, dim=0)
    counts = torch.bincount(ids, minlength=num_segments)
    ends = torch.cumsum(counts, 0)
    starts = ends - counts
    zero = torch.zeros((1,) + tuple(v.shape[1:]), dtype=v.dtype, device=v.device)
    csz = torch.cat([zero, cs], 0)
    return (csz[ends] - csz[starts]).to(values.dtype)
