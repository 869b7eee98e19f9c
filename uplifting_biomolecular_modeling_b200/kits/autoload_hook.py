"""The ``.pth`` hook of the kits and the step of ``install`` that places it.

``run.sh install --pth-dir D`` writes ``<kit>_opt_autoload.pth`` into the site directory D (a directory on which
Python processes ``.pth`` files: ``site-packages`` of the environment, or one added with ``site.addsitedir``).  The
file holds one line that reads the kit's variable first and imports this module only when the variable is set, so
a process without ``<KIT>_OPT`` loads nothing of the package.  With the variable set, :func:`install_for`
installs the meta-path finder of :mod:`core.autoload`: the first import of one of the kit's trigger modules (the
model family the kit serves) calls ``enable(mode)`` for the kit; every failure there is one ``NOT ACTIVE`` line
and exit 3.  Reference: the PEP 517 build backend that ships ``<pkg>_autoload.pth`` at the wheel root
(common/opt_core/kit_template/_build_backend.py) and ``<kit>_opt/_autoload.py`` of every kit.
"""
from __future__ import annotations

import os
import sys
import types
from typing import Optional

PACKAGE = "uplifting_biomolecular_modeling_b200"

# model-family modules whose first import is "the upstream tool is being loaded" for a kit of that family
TRIGGERS = {
    "cofold": (f"{PACKAGE}.models.cofold", f"{PACKAGE}.api"),
    "design": (f"{PACKAGE}.models.design", f"{PACKAGE}.models.cofold"),
    "evo2": (f"{PACKAGE}.models.evo2",),
    "protein_lm": (f"{PACKAGE}.models.plm",),
    "genomic_track": (f"{PACKAGE}.models.genomics",),
}


def pth_name(kit: str) -> str:
    return f"{kit}_opt_autoload.pth"


def pth_line(kit: str, env: str) -> str:
    """One ``import`` statement (the only kind of line ``site`` executes): cheap when the variable is unset."""
    return (f"import os, sys; os.environ.get({env!r}) and "
            f"__import__({PACKAGE + '.kits.autoload_hook'!r}, fromlist=['install_for']).install_for({kit!r})\n")


def place_pth(kit: str, site_dir: str, repo_root: Optional[str] = None) -> str:
    """Write the kit's ``.pth`` file into ``site_dir``.  The first line puts the repository root on ``sys.path`` (the
    package is used in-tree, not installed), the second is the hook.  Returns the path."""
    from .registry import get
    spec = get(kit)
    root = repo_root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    os.makedirs(site_dir, exist_ok=True)
    path = os.path.join(site_dir, pth_name(kit))
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        f.write(root + "\n")
        f.write(pth_line(kit, spec.env))
    os.replace(tmp, path)
    return path


def install_for(kit: str):
    """Called from the ``.pth`` line.  Installs the finder (or prints NOT ACTIVE and exits 3 for an unknown mode)."""
    from ..core import autoload
    from .registry import get
    spec = get(kit)
    shim_name = f"{PACKAGE}.kits._enable_{kit}"
    if shim_name not in sys.modules:
        from . import base
        shim = types.ModuleType(shim_name)
        shim.enable = lambda mode, strict=True, trigger=None, _k=kit: base.enable(_k, mode, strict=strict,
                                                                                  trigger=trigger)
        sys.modules[shim_name] = shim
    a = autoload.AutoloadSpec(spec.tag, spec.env, shim_name, TRIGGERS.get(spec.family, ()), tuple(spec.modes))
    return autoload.install(a)
