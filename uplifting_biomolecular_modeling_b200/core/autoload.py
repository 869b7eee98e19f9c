"""In-process activation: ``<KIT>_OPT=<mode> python user_script.py``.

A ``.pth`` file runs :func:`install` at interpreter start.  ``install`` reads the kit's variable and,
only when it is set, inserts a meta-path :class:`Finder` that waits for the first import of a
*trigger* module (the upstream tool's model package), lets the module body run, and then calls
``<kit package>.enable(mode, strict=True, trigger=<name>)``.  Any failure - unknown mode, a gate
that fails, a lever that cannot run - prints exactly one ``NOT ACTIVE`` line and exits 3; the process
never continues on stock code under the mode's label.  With the variable unset nothing is imported
and nothing is patched.  Reference: common/opt_core/opt_core/autoload.py:56,166,211,256,430.
"""
from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import os
import sys
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Mapping, Optional, Sequence, Tuple

from . import report


@dataclass
class AutoloadSpec:
    kit: str                      # tag of the lines, e.g. "boltz2-opt"
    env: str                      # variable that selects the mode, e.g. "BOLTZ2_OPT"
    package: str                  # kit package that offers enable(mode, strict, trigger)
    triggers: Tuple[str, ...]     # modules whose first import fires activation
    modes: Tuple[str, ...] = ("off", "exact", "fast", "big")
    exit_fn: Callable[[int], None] = sys.exit


@dataclass
class AttrPatch:
    """Replace one attribute of a module when (and only when) that module is imported."""
    module: str
    attr: str
    make: Callable[[object], object]     # old value -> new value
    applied: bool = False


class _Loader(importlib.abc.Loader):
    def __init__(self, inner, after: Callable[[object], None]):
        self._inner, self._after = inner, after

    def create_module(self, spec):
        cm = getattr(self._inner, "create_module", None)
        return cm(spec) if cm else None

    def exec_module(self, module):
        self._inner.exec_module(module)
        self._after(module)

    def __getattr__(self, name):
        return getattr(self._inner, name)


class Finder(importlib.abc.MetaPathFinder):
    """Wraps the loader of trigger modules; everything else is left to the normal finders."""

    def __init__(self, spec: AutoloadSpec, mode: str):
        self.spec, self.mode = spec, mode
        self.fired = False
        self.patches: List[AttrPatch] = []
        self._busy = False

    def find_spec(self, fullname, path=None, target=None):
        wanted = (fullname in self.spec.triggers and not self.fired) or any(
            p.module == fullname and not p.applied for p in self.patches)
        if not wanted or self._busy:
            return None
        self._busy = True
        try:
            real = importlib.util.find_spec(fullname)
        except (ImportError, ValueError):
            real = None
        finally:
            self._busy = False
        if real is None or real.loader is None:
            return None
        real.loader = _Loader(real.loader, lambda module, n=fullname: self._after_import(n, module))
        return real

    def _after_import(self, name: str, module) -> None:
        for p in self.patches:
            if p.module == name and not p.applied:
                setattr(module, p.attr, p.make(getattr(module, p.attr, None)))
                p.applied = True
        if name in self.spec.triggers and not self.fired:
            self.fired = True
            fire(self.spec, self.mode, trigger=name)


def fire(spec: AutoloadSpec, mode: str, trigger: Optional[str] = None) -> None:
    """Call the kit's ``enable``; turn every failure into one NOT ACTIVE line and exit 3."""
    try:
        pkg = importlib.import_module(spec.package)
        pkg.enable(mode, strict=True, trigger=trigger)
    except SystemExit:
        raise
    except BaseException as e:  # noqa: BLE001
        reason = f"{type(e).__name__}: {e}" if str(e) else type(e).__name__
        report.emit(report.not_active_line(spec.kit, reason, f"mode={mode} trigger={trigger or 'none'}"))
        spec.exit_fn(report.EXIT_NOT_ACTIVE)


def install(spec: AutoloadSpec, environ: Optional[Mapping[str, str]] = None,
            meta_path: Optional[list] = None) -> Optional[Finder]:
    """Called from the kit's ``.pth`` hook.  Returns the finder, or None when the variable is unset
    (stock process: nothing installed)."""
    env = os.environ if environ is None else environ
    mode = (env.get(spec.env) or "").strip()
    if not mode or mode == "off":
        return None
    if mode not in spec.modes:
        report.emit(report.not_active_line(spec.kit, f"unknown mode {mode!r} in {spec.env}; known: "
                                                     f"{', '.join(spec.modes)}"))
        spec.exit_fn(report.EXIT_NOT_ACTIVE)
        return None
    mp = sys.meta_path if meta_path is None else meta_path
    for f in mp:
        if isinstance(f, Finder) and f.spec.kit == spec.kit:
            return f
    finder = Finder(spec, mode)
    mp.insert(0, finder)
    # a trigger that is already imported fires at once
    for t in spec.triggers:
        if t in sys.modules and not finder.fired:
            finder.fired = True
            fire(spec, mode, trigger=t)
    return finder


def patch_attr_at_import(finder: Finder, module: str, attr: str, make: Callable[[object], object]) -> AttrPatch:
    """Replace ``module.attr`` when ``module`` is imported (at once if it already is)."""
    p = AttrPatch(module, attr, make)
    if module in sys.modules:
        m = sys.modules[module]
        setattr(m, attr, make(getattr(m, attr, None)))
        p.applied = True
    finder.patches.append(p)
    return p


def pth_line(package: str) -> str:
    """Content of ``<package>_autoload.pth``: one import line that runs the kit's hook."""
    return f"import {package}._autoload\n"
