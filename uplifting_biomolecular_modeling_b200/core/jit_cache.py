"""Build-cache location keyed by the software stack: ``torch<ver>-cu<cuda>-sm<cc>``.

Root: ``MODEL_OPT_JIT_ROOT`` when set, else ``${TMPDIR:-/tmp}/model_opt_jit-uid<uid>``.  The key keeps
objects built for one stack from being loaded under another.  Reference: common/opt_core/opt_core/jit_cache.py:124."""
from __future__ import annotations

import os
import tempfile
from typing import Mapping, Optional


def stack_key(torch_version: Optional[str] = None, cuda: Optional[str] = None, sm: Optional[str] = None) -> str:
    if torch_version is None or cuda is None:
        try:
            import torch
            torch_version = torch_version or torch.__version__.split("+")[0]
            cuda = cuda or (torch.version.cuda or "none")
        except Exception:  # noqa: BLE001
            torch_version, cuda = torch_version or "none", cuda or "none"
    sm = sm or "100a"
    return f"torch{torch_version}-cu{str(cuda).replace('.', '')}-sm{str(sm).replace('sm', '').replace('.', '')}"


def root(environ: Optional[Mapping[str, str]] = None) -> str:
    env = os.environ if environ is None else environ
    r = env.get("MODEL_OPT_JIT_ROOT")
    if r:
        return r
    base = env.get("TMPDIR") or tempfile.gettempdir()
    return os.path.join(base, f"model_opt_jit-uid{os.getuid()}")


def cache_dir(kit: str, key: Optional[str] = None, environ: Optional[Mapping[str, str]] = None,
              create: bool = True) -> str:
    d = os.path.join(root(environ), kit, key or stack_key())
    if create:
        os.makedirs(d, exist_ok=True)
    return d
