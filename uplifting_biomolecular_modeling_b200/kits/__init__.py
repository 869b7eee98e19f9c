"""Kits: the per-tool public surface (``run.sh``, ``<KIT>_OPT``, ``enable()``, ACTIVE / NOT ACTIVE lines)."""
from .base import Activation, ActivationError, enable, status  # noqa: F401
from .registry import REGISTRY, KitSpec, get, names  # noqa: F401
