"""Content-addressed memo of an expensive host-side build (features, MSA parses, conformers, embeddings).

``Memo(name).get_or_build(parts, build)`` returns ``build()``'s value for the key ``digest(parts)``, computing it
once per key per process (and once per directory with ``disk_dir``).  ``parts`` names every input that
determines the value (input bytes or their file digest, seed, builder name and version, settings); an input the
digest cannot canonicalise is refused by type name, and a deliberate bypass is counted under its reason so
that nothing uncached is silent.  Reference: common/opt_core/opt_core/host/memo.py.
"""
from __future__ import annotations

import hashlib
import os
import pickle
import struct
from collections import OrderedDict
from typing import Any, Callable, Dict, Mapping, Optional


class Undigestible(TypeError):
    pass


class MemoMismatch(RuntimeError):
    """A verification rebuild disagreed with the cached value."""


def _feed(h, obj) -> None:
    if obj is None:
        h.update(b"N")
    elif isinstance(obj, bool):
        h.update(b"B1" if obj else b"B0")
    elif isinstance(obj, int):
        h.update(b"I" + str(obj).encode())
    elif isinstance(obj, float):
        h.update(b"F" + struct.pack("<d", obj))
    elif isinstance(obj, str):
        b = obj.encode()
        h.update(b"S" + str(len(b)).encode() + b":" + b)
    elif isinstance(obj, (bytes, bytearray, memoryview)):
        b = bytes(obj)
        h.update(b"Y" + str(len(b)).encode() + b":" + b)
    elif isinstance(obj, (list, tuple)):
        h.update(b"L" + str(len(obj)).encode())
        for x in obj:
            _feed(h, x)
    elif isinstance(obj, Mapping):
        h.update(b"M" + str(len(obj)).encode())
        for k in sorted(obj, key=lambda k_: (type(k_).__name__, str(k_))):
            _feed(h, k)
            _feed(h, obj[k])
    elif hasattr(obj, "tobytes") and hasattr(obj, "shape") and hasattr(obj, "dtype"):     # numpy / torch cpu
        arr = obj.detach().cpu().numpy() if hasattr(obj, "detach") else obj
        h.update(b"A" + str(arr.dtype).encode() + str(tuple(arr.shape)).encode())
        h.update(arr.tobytes())
    else:
        raise Undigestible(f"undigestible:{type(obj).__name__}")


def digest(obj) -> str:
    h = hashlib.sha256()
    _feed(h, obj)
    return h.hexdigest()


def file_digest(path: str, chunk: int = 1 << 20) -> str:
    """sha256 of a file's bytes: the part to key on for an input file (never its path or mtime)."""
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


class Memo:
    def __init__(self, name: str, max_items: int = 64, disk_dir: Optional[str] = None, verify_every: int = 0,
                 equal: Optional[Callable[[Any, Any], bool]] = None):
        self.name, self.max_items, self.disk_dir, self.verify_every = name, max_items, disk_dir, verify_every
        self.equal = equal or (lambda a, b: digest(a) == digest(b))
        self._mem: "OrderedDict[str, Any]" = OrderedDict()
        self.stats: Dict[str, int] = {"hit": 0, "disk_hit": 0, "build": 0, "verified": 0}
        self.bypasses: Dict[str, int] = {}
        if disk_dir:
            os.makedirs(disk_dir, exist_ok=True)

    def _path(self, key: str) -> str:
        return os.path.join(self.disk_dir, f"{self.name}-{key}.pkl")

    def get_or_build(self, parts: Mapping[str, Any], build: Callable[[], Any], bypass: Optional[str] = None):
        if bypass is not None:
            self.bypasses[bypass] = self.bypasses.get(bypass, 0) + 1
            return build()
        key = digest(parts)
        if key in self._mem:
            self._mem.move_to_end(key)
            self.stats["hit"] += 1
            val = self._mem[key]
            if self.verify_every and self.stats["hit"] % self.verify_every == 0:
                fresh = build()
                self.stats["verified"] += 1
                if not self.equal(val, fresh):
                    raise MemoMismatch(f"memo {self.name}: cached value of {key[:12]} differs from a rebuild")
            return val
        if self.disk_dir and os.path.exists(self._path(key)):
            with open(self._path(key), "rb") as f:
                val = pickle.load(f)
            self.stats["disk_hit"] += 1
        else:
            val = build()
            self.stats["build"] += 1
            if self.disk_dir:
                tmp = self._path(key) + f".tmp{os.getpid()}"
                with open(tmp, "wb") as f:
                    pickle.dump(val, f, protocol=4)
                os.replace(tmp, self._path(key))
        self._mem[key] = val
        while len(self._mem) > self.max_items:
            self._mem.popitem(last=False)
        return val

    def words(self):
        w = [f"memo_{self.name}=hit:{self.stats['hit']},disk:{self.stats['disk_hit']},build:{self.stats['build']}"]
        w += [f"memo_{self.name}_bypass={r}:{n}" for r, n in sorted(self.bypasses.items())]
        return w
