"""Build the sm_100a kernel library in-tree.

Every ``*.cu`` under ``ops/csrc`` is compiled with
``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo`` and linked into one shared object,
``ops/_lib/libubm_sm100.so``, which exports a plain C ABI (``extern "C"`` functions taking raw
device pointers and a stream handle).  The library links the static CUDA runtime and looks the
driver's tensor-map encoder up at first use, so it loads on a machine without a GPU driver.

The reference compiles its CUDA members at first use with NVRTC or ships arch-keyed cubins
(common/opt_core/opt_core/kernels/triattn_exact/README.md:27,
common/opt_core/opt_core/kernels/trimul/native/DESIGN.md:90-92); here there is one arch and one
library, built ahead of time.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIBDIR = Path(__file__).resolve().parent / "_lib"
LIBNAME = "libubm_sm100.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found (set NVCC)")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def library_path() -> Path:
    return LIBDIR / LIBNAME


def is_current() -> bool:
    stamp = LIBDIR / "build.sha256"
    lib = library_path()
    if not lib.exists() or not stamp.exists():
        return False
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    return stamp.read_text().strip() == _digest(deps)


def _compile_one(src: Path, obj: Path, log: Path) -> None:
    cmd = [_nvcc(), *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")


def build(force: bool = False, verbose: bool = True) -> Path:
    """Compile and link; returns the library path. No-op when sources are unchanged."""
    LIBDIR.mkdir(parents=True, exist_ok=True)
    if not force and is_current():
        return library_path()
    objdir = LIBDIR / "obj"
    objdir.mkdir(exist_ok=True)
    srcs = sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        futs = {ex.submit(_compile_one, s, objdir / (s.stem + ".o"), objdir / (s.stem + ".log")): s for s in srcs}
        for f in concurrent.futures.as_completed(futs):
            f.result()
            if verbose:
                print(f"[ubm-build] compiled {futs[f].name}", file=sys.stderr)
    objs = [str(objdir / (s.stem + ".o")) for s in srcs]
    cmd = [_nvcc(), "-shared", "-o", str(library_path()), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))
    (LIBDIR / "build.sha256").write_text(_digest(deps) + "\n")
    if verbose:
        print(f"[ubm-build] linked {library_path()}", file=sys.stderr)
    return library_path()


def ptxas_report() -> dict:
    """Registers / spills / shared memory per kernel, parsed from the last build's logs."""
    out = {}
    objdir = LIBDIR / "obj"
    for log in sorted(objdir.glob("*.log")):
        cur = None
        for line in log.read_text().splitlines():
            if "Compiling entry function" in line:
                cur = line.split("'")[1]
            elif "Used" in line and cur:
                out[cur] = line.split(":", 1)[1].strip()
            elif "spill" in line and cur:
                out[cur + ":frame"] = line.strip()
    return out


if __name__ == "__main__":
    build(force="--force" in sys.argv)
    for k, v in ptxas_report().items():
        print(k, "->", v)
