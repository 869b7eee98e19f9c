"""Layering and hygiene of the source tree."""
import os
import re
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "uplifting_biomolecular_modeling_b200")


def _sources(exts):
    for base, dirs, files in os.walk(ROOT):
        dirs[:] = [d for d in dirs if d not in (".git", "_work", "gpurun_out", "baseline", "__pycache__", "_lib")]
        for f in files:
            if f.endswith(exts):
                yield os.path.join(base, f)


def test_contract_runtime_imports_without_the_tensor_library():
    mods = sorted(f[:-3] for f in os.listdir(os.path.join(PKG, "core")) if f.endswith(".py") and f != "__init__.py")
    code = ("import sys\n" + "".join(f"import uplifting_biomolecular_modeling_b200.core.{m}\n" for m in mods) +
            "print(sorted(m for m in ('torch', 'numpy', 'triton') if m in sys.modules))")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip() == "[]", r.stdout


def test_nothing_committed_depends_on_scratch_or_compat_layers():
    bad = []
    for path in _sources((".py",)):
        if os.path.basename(path) == "test_layering_cpu.py":
            continue
        text = open(path, errors="replace").read()
        if re.search(r"^\s*(import|from)\s+_work\b|[\"']_work/", text, re.M):
            bad.append((path, "_work"))
        if re.search(r"^\s*(import|from)\s+(triton|tilelang)\b", text, re.M) or "torch.compile(" in text:
            bad.append((path, "compat layer"))
    assert not bad, bad


def test_every_wait_in_the_tensor_core_kernels_is_bounded():
    """Spin loops on barriers go through the bounded helpers of sm100.cuh (time limit + status word)."""
    csrc = os.path.join(PKG, "ops", "csrc")
    for f in os.listdir(csrc):
        if not f.endswith(".cu"):
            continue
        text = open(os.path.join(csrc, f)).read()
        assert "mbarrier.try_wait" not in text and "mbarrier.test_wait" not in text, \
            f"{f}: raw barrier wait outside the bounded helper"
    helper = open(os.path.join(csrc, "sm100.cuh")).read()
    assert "globaltimer" in helper and "try_wait" in helper


def test_pair_index_products_are_64_bit():
    """N * N * 128 passes 2^31 at N = 4096: every product of two token extents in kernel code is widened first."""
    csrc = os.path.join(PKG, "ops", "csrc")
    rx = re.compile(r"\bN\s*\*\s*(N|Np)\b|\bNp\s*\*\s*N\b")
    bad = []
    for f in sorted(os.listdir(csrc)):
        if not f.endswith((".cu", ".cuh")):
            continue
        for n, line in enumerate(open(os.path.join(csrc, f)), 1):
            code = line.split("//")[0]
            if rx.search(code) and not re.search(r"long long|size_t|int64_t|uint64_t", code):
                bad.append(f"{f}:{n}: {code.strip()}")
    assert not bad, bad
