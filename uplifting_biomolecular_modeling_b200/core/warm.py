"""Early heavy imports: start importing the modules a command will need on a helper thread while the command
line is still being parsed and files are being read, and report what the overlap bought.
Reference: common/opt_core/opt_core/warm.py:69."""
from __future__ import annotations

import importlib
import threading

from . import pystack
import time
from typing import Dict, Optional, Sequence


class Warm:
    def __init__(self, modules: Sequence[str]):
        self.modules = list(modules)
        self.seconds: Dict[str, float] = {}
        self.errors: Dict[str, str] = {}
        self._thread: Optional[threading.Thread] = None

    def _run(self) -> None:
        for m in self.modules:
            t0 = time.perf_counter()
            try:
                # imports run from a frame larger than a stack chunk (see core.pystack): their cost must not
                # depend on the depth this thread happens to be at
                pystack.roomy_call(importlib.import_module, m)
            except Exception as e:                      # a failed warm-up is not an error: the real import reports it
                self.errors[m] = f"{type(e).__name__}: {e}"
            self.seconds[m] = time.perf_counter() - t0

    def start(self) -> "Warm":
        self._thread = threading.Thread(target=self._run, name="warm-imports", daemon=True)
        self._thread.start()
        return self

    def join(self, timeout: Optional[float] = None) -> Dict[str, float]:
        if self._thread is not None:
            self._thread.join(timeout)
        return dict(self.seconds)


def warm(modules: Sequence[str]) -> Warm:
    return Warm(modules).start()
