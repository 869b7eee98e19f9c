"""Where the tree is: repository root, kit directories, the package directory.
Reference: common/opt_core/opt_core/home.py:24."""
from __future__ import annotations

import os
from typing import List, Optional

PACKAGE_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REPO_ROOT = os.path.dirname(PACKAGE_DIR)


def kits_root() -> str:
    return os.path.join(REPO_ROOT, "kits")


def kit_dir(kit: str) -> str:
    return os.path.join(kits_root(), kit)


def list_kit_dirs() -> List[str]:
    r = kits_root()
    if not os.path.isdir(r):
        return []
    return sorted(d for d in os.listdir(r) if os.path.isfile(os.path.join(r, d, "run.sh")))


def config_path(kit: str, card: str) -> Optional[str]:
    p = os.path.join(kit_dir(kit), "configs", f"{card}.env")
    return p if os.path.isfile(p) else None
