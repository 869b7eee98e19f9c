"""``opt_manifest.json``: what a run engaged, written atomically beside its outputs.

Fields: kit, mode and its source, levers applied / skipped with reasons, evidence words, the
exit verdict, the GPU, versions, per-lever ledger counts.  Reference: common/opt_core/opt_core/manifest.py:17,48,75.
"""
from __future__ import annotations

import json
import os
import tempfile
import time
from typing import Mapping, Optional

MANIFEST_NAME = "opt_manifest.json"
SCHEMA = 1


def build(kit: str, mode: str, mode_source: str, levers_on, levers_skipped: Optional[Mapping[str, str]] = None,
          words=(), verdict: Optional[Mapping] = None, gpu=None, versions: Optional[Mapping] = None,
          ledgers: Optional[Mapping] = None, extra: Optional[Mapping] = None) -> dict:
    m = {"schema": SCHEMA, "kit": kit, "mode": mode, "mode_source": mode_source, "levers_on": list(levers_on),
         "levers_skipped": dict(levers_skipped or {}), "words": list(words), "verdict": dict(verdict or {}),
         "gpu": gpu, "versions": dict(versions or {}), "ledgers": dict(ledgers or {}),
         "written_unix": round(time.time(), 3)}
    if extra:
        m.update(extra)
    return m


def write(dirpath, manifest: Mapping, name: str = MANIFEST_NAME) -> str:
    """Atomic write (temp file in the same directory, fsync, rename)."""
    os.makedirs(dirpath, exist_ok=True)
    fd, tmp = tempfile.mkstemp(prefix="." + name + ".", dir=dirpath)
    try:
        with os.fdopen(fd, "w", encoding="utf-8") as f:
            json.dump(manifest, f, indent=1, sort_keys=True, default=str)
            f.write("\n")
            f.flush()
            os.fsync(f.fileno())
        path = os.path.join(dirpath, name)
        os.replace(tmp, path)
        return path
    except BaseException:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise


def read(dirpath, name: str = MANIFEST_NAME) -> Optional[dict]:
    p = os.path.join(dirpath, name)
    try:
        with open(p, "r", encoding="utf-8") as f:
            return json.load(f)
    except (OSError, ValueError):
        return None
