"""Proof that an ``off`` process is clean: no kit variables in its environment, no kit module
imported, no activation finder on the meta path.  The ``off`` route of a kit runs the stock tool in a
child process and asks the child for this proof before trusting its numbers.
Reference: common/opt_core/opt_core/stock_proof.py:121."""
from __future__ import annotations

import os
import sys
from typing import Iterable, List, Mapping, Optional


def env_proof(kit_env_prefixes: Iterable[str], kit_modules: Iterable[str],
              environ: Optional[Mapping[str, str]] = None, modules: Optional[Mapping[str, object]] = None,
              meta_path: Optional[list] = None) -> dict:
    env = os.environ if environ is None else environ
    mods = sys.modules if modules is None else modules
    mp = sys.meta_path if meta_path is None else meta_path
    prefixes = tuple(kit_env_prefixes)
    kmods = tuple(kit_modules)
    env_hits = sorted(k for k in env if k.startswith(prefixes) and (env.get(k) or "").strip() not in ("", "off"))
    mod_hits = sorted(m for m in mods if any(m == k or m.startswith(k + ".") for k in kmods))
    finder_hits = [type(f).__name__ for f in mp if type(f).__module__.endswith("core.autoload")]
    return {"clean": not (env_hits or mod_hits or finder_hits), "env": env_hits, "modules": mod_hits,
            "finders": finder_hits}


def proof_line(tag: str, proof: Mapping) -> str:
    from . import report
    return report.line(tag, "STOCK", ("clean", proof["clean"]), ("env", proof["env"]), ("modules", proof["modules"]),
                       ("finders", proof["finders"]))
