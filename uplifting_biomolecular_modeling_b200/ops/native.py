"""ctypes face of the sm_100a kernel library.

The library exports a C ABI; this module loads it, declares argument types and offers helpers
to pass torch tensors (data pointers) and the current CUDA stream.  On a machine with a GPU a
missing library is an error (never a silent eager fallback): callers that want the kernels call
:func:`lib` and get ``NativeUnavailable`` with the reason.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path
from typing import Optional

from . import build as _build


class NativeUnavailable(RuntimeError):
    """The kernel library cannot be loaded (not built, or load error)."""


class KernelFault(RuntimeError):
    """A kernel reported a non-zero status word or an entry point returned an error code."""


_LOCK = threading.Lock()
_LIB = None

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float

_SIGNATURES = {
    "ubm_gemm_bf16": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                      c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_float,
                      c_void_p, c_void_p],
    "ubm_template_embed": [c_void_p] * 11 + [c_int, c_int, c_void_p],
    "ubm_template_tail": [c_void_p, c_void_p, c_int, c_ll, c_int, c_void_p],
    "ubm_gemm_bf16_ex": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                         c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_float,
                         c_ll, c_ll, c_ll, c_void_p, c_ll, c_int, c_int, c_void_p, c_void_p],
}

ERROR_NAMES = {0: "ok", -1: "bad argument", -2: "driver entry point / tensor map", -3: "launch failed",
               -4: "workspace too large"}
STATUS_NAMES = {0: "ok", 1: "mbarrier wait ran out", 2: "peer flag wait ran out", 3: "bad argument"}


def library_path() -> Path:
    env = os.environ.get("UBM_B200_LIB")
    return Path(env) if env else _build.library_path()


def declare(name: str, argtypes) -> None:
    """Register the signature of an exported symbol (used by op modules beside their kernels)."""
    _SIGNATURES[name] = list(argtypes)
    if _LIB is not None:
        _LIB._cache.pop(name, None)


def lib(build_if_missing: bool = False):
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        path = library_path()
        if not path.exists():
            if build_if_missing:
                _build.build()
            else:
                raise NativeUnavailable(f"kernel library not built: {path} (run python -m "
                                        f"uplifting_biomolecular_modeling_b200.ops.build)")
        try:
            handle = ctypes.CDLL(str(path))
        except OSError as e:  # pragma: no cover - depends on the machine
            raise NativeUnavailable(f"cannot load {path}: {e}") from e
        for name, argtypes in _SIGNATURES.items():
            if hasattr(handle, name):
                fn = getattr(handle, name)
                fn.argtypes = argtypes
                fn.restype = c_int
        _LIB = _LibProxy(handle)
        return _LIB


class _LibProxy:
    """Attribute access returns counted callables; unknown symbols raise AttributeError as ctypes does."""

    def __init__(self, handle):
        self._handle = handle
        self._cache = {}

    def __getattr__(self, name):
        c = self._cache.get(name)
        if c is None:
            fn = getattr(self._handle, name)
            if name in _SIGNATURES:
                fn.argtypes = _SIGNATURES[name]
                fn.restype = c_int
            c = _Counted(fn, name)
            self._cache[name] = c
        return c


class _Counted:
    """Callable proxy of an exported symbol that counts launches (one call = one or more kernels)."""

    __slots__ = ("fn", "name")

    def __init__(self, fn, name):
        self.fn, self.name = fn, name

    def __call__(self, *a):
        _COUNTS[self.name] = _COUNTS.get(self.name, 0) + 1
        return self.fn(*a)


_COUNTS: dict = {}


def launch_count() -> int:
    """Entry-point calls since the last reset (each is one kernel launch of this library)."""
    return sum(_COUNTS.values())


def add_launches(n: int, name: str = "graph_replay") -> None:
    """Account for kernels of this library launched by a CUDA-graph replay (n per replay)."""
    _COUNTS[name] = _COUNTS.get(name, 0) + int(n)


def launch_counts() -> dict:
    return dict(_COUNTS)


def reset_launch_count() -> None:
    _COUNTS.clear()


def available() -> bool:
    try:
        lib()
        return True
    except NativeUnavailable:
        return False


def ptr(t) -> int:
    """Device pointer of a tensor (0 for None)."""
    return 0 if t is None else t.data_ptr()


def current_stream(device=None) -> int:
    import torch
    return torch.cuda.current_stream(device).cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise KernelFault(f"{what}: entry point returned {rc} ({ERROR_NAMES.get(rc, 'unknown')})")


# ---- per-device status word ----------------------------------------------------------------
_STATUS = {}


def status_tensor(device):
    """A 4 x uint32 device tensor that kernels write their error status into."""
    import torch
    dev = torch.device(device)
    key = (dev.type, dev.index if dev.index is not None else torch.cuda.current_device())
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=dev)
        _STATUS[key] = t
    return t


def read_status(device, reset: bool = True):
    """Synchronise and return (code, where, block, aux)."""
    t = status_tensor(device)
    vals = tuple(int(v) & 0xFFFFFFFF for v in t.cpu().tolist())
    if reset and vals[0] != 0:
        t.zero_()
    return vals


def raise_on_status(device, what: str = "kernel") -> None:
    code, where, block, aux = read_status(device)
    if code != 0:
        raise KernelFault(f"{what}: device status {code} ({STATUS_NAMES.get(code, '?')}) at site {where}, "
                          f"block {block}, aux {aux}")
