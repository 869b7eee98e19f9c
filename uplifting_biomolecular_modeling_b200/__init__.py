"""B200-native inference framework for biomolecular models.

Importing the package imports nothing heavy: sub-packages are resolved lazily (PEP 562) so that a
process started under a kit's activation hook pays for torch / CUDA only when a model is built
(same rule as the reference core: common/opt_core/opt_core/__init__.py:58-88).
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_SUBPACKAGES = ("core", "ops", "models", "parallel", "mem", "capture", "kits", "utils")


def __getattr__(name):
    if name in _SUBPACKAGES:
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)


def __dir__():
    return sorted(list(globals()) + list(_SUBPACKAGES))
