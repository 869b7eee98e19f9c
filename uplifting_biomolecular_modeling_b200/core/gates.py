"""Named pre-flight checks ("gates") with a verdict and evidence words.

A gate answers one question about the machine or the installation before a mode engages: which
GPU is present (``nvidia-smi`` first, torch second, so that a probe does not initialise CUDA),
whether a package is at its pinned version, whether carried files match their ``SHA256SUMS``,
whether a prebuilt binary matches its recorded digest before it is loaded.  A failing mandatory
gate makes the kit print ``NOT ACTIVE`` and exit 3; a lever that cannot run where it was asked to
raises an exception carrying ``cannot_run = True``.  Reference: common/opt_core/opt_core/gates.py:57,
74,161,238,413,505.
"""
from __future__ import annotations

import hashlib
import os
import re
import shutil
import subprocess
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

from . import report


class CannotRun(RuntimeError):
    """A lever's mechanism fails where it was asked to run; the mode is refused by name."""

    cannot_run = True


def cannot_run(exc: BaseException) -> BaseException:
    """Mark an existing exception as a cannot-run event."""
    try:
        exc.cannot_run = True  # type: ignore[attr-defined]
    except Exception:  # noqa: BLE001
        pass
    return exc


def is_cannot_run(exc: BaseException) -> bool:
    return bool(getattr(exc, "cannot_run", False))


@dataclass
class Gate:
    name: str
    ok: bool
    detail: str = ""
    words: Tuple[str, ...] = ()
    mandatory: bool = True

    def line(self, tag: str) -> str:
        return report.line(tag, "GATE", ("name", self.name), ("verdict", "pass" if self.ok else "fail"),
                           ("detail", report.token(self.detail) if self.detail else "none"))


def run_gates(checks: Sequence[Callable[[], Gate]]) -> Tuple[bool, List[Gate]]:
    """Run every check (a failing check never hides the later ones); ok = all mandatory gates passed."""
    gates: List[Gate] = []
    for c in checks:
        try:
            g = c()
        except Exception as e:  # noqa: BLE001
            g = Gate(getattr(c, "__name__", "gate"), False, f"{type(e).__name__}: {e}")
        gates.append(g)
    return all(g.ok or not g.mandatory for g in gates), gates


def first_failure(gates: Iterable[Gate]) -> Optional[Gate]:
    for g in gates:
        if not g.ok and g.mandatory:
            return g
    return None


# ----------------------------------------------------------------------------- GPU probes
GPU_CLASSES: Dict[str, Dict[str, object]] = {
    # class word -> (substring of the product name, sm, nominal memory in MiB)
    "b200": {"match": "B200", "sm": "sm100", "mem_mib": 183359},
    "b300": {"match": "B300", "sm": "sm103", "mem_mib": 275000},
    "gb200": {"match": "GB200", "sm": "sm100", "mem_mib": 188000},
    "h100": {"match": "H100", "sm": "sm90", "mem_mib": 81559},
    "h200": {"match": "H200", "sm": "sm90", "mem_mib": 143771},
    "a100": {"match": "A100", "sm": "sm80", "mem_mib": 81920},
}


def nvidia_smi_probe(run=subprocess.run, which=shutil.which) -> List[dict]:
    """``[{index, name, cc, sm, mem_mib}]`` from nvidia-smi; [] when it is absent or fails."""
    exe = which("nvidia-smi")
    if not exe:
        return []
    try:
        res = run([exe, "--query-gpu=index,name,compute_cap,memory.total", "--format=csv,noheader,nounits"],
                  capture_output=True, text=True, timeout=20)
    except Exception:  # noqa: BLE001
        return []
    if getattr(res, "returncode", 1) != 0:
        return []
    out = []
    for ln in res.stdout.strip().splitlines():
        parts = [p.strip() for p in ln.split(",")]
        if len(parts) < 4:
            continue
        cc = parts[2]
        out.append({"index": int(parts[0]) if parts[0].isdigit() else len(out), "name": parts[1], "cc": cc,
                    "sm": "sm" + cc.replace(".", ""), "mem_mib": int(float(parts[3])) if parts[3] else None})
    return out


def torch_probe() -> List[dict]:
    try:
        import torch
        if not torch.cuda.is_available():
            return []
        out = []
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out.append({"index": i, "name": p.name, "cc": f"{p.major}.{p.minor}", "sm": f"sm{p.major}{p.minor}",
                        "mem_mib": p.total_memory // (1 << 20)})
        return out
    except Exception:  # noqa: BLE001
        return []


def probe_gpus() -> List[dict]:
    return nvidia_smi_probe() or torch_probe()


def gpu_class(name: str) -> Optional[str]:
    # longest match first so that GB200 is not read as B200
    for word, spec in sorted(GPU_CLASSES.items(), key=lambda kv: -len(str(kv[1]["match"]))):
        if str(spec["match"]).lower() in (name or "").lower():
            return word
    return None


def gpu_gate(min_sm: int = 100, target: Optional[str] = None, probe: Callable[[], List[dict]] = probe_gpus,
             n_required: int = 1) -> Gate:
    """At least ``n_required`` GPUs of compute capability >= min_sm; an unlisted card is a word, not a failure."""
    gpus = probe()
    if len(gpus) < n_required:
        return Gate("gpu", False, f"{len(gpus)} GPU(s) visible, {n_required} needed")
    words = []
    for g in gpus[:n_required]:
        sm = int(re.sub(r"\D", "", str(g["sm"])) or 0)
        if sm < min_sm:
            return Gate("gpu", False, f"{g['name']} is {g['sm']}; this build needs sm{min_sm} (tcgen05/TMEM)")
        cls = gpu_class(str(g["name"]))
        if cls is None:
            words.append(report.word("card", "uncertified", g["name"], f"{g['mem_mib']}MiB"))
        elif target and cls != target:
            words.append(report.word("card", "other_than_config", cls, target))
    return Gate("gpu", True, report.gpu_label(gpus[0]), tuple(dict.fromkeys(words)))


# ----------------------------------------------------------------------------- version / pin gates
def _ver_tuple(v: str) -> Tuple[int, ...]:
    return tuple(int(x) for x in re.findall(r"\d+", v)[:4])


def version_gate(name: str, found: Optional[str], minimum: Optional[str] = None, exact: Optional[str] = None,
                 mandatory: bool = True) -> Gate:
    if found is None:
        return Gate(f"version:{name}", False, "not installed", mandatory=mandatory)
    if exact is not None and found != exact:
        return Gate(f"version:{name}", not mandatory, f"{found}!={exact}",
                    (report.word("stack", "drift", f"{name}:{found}!={exact}"),), mandatory)
    if minimum is not None and _ver_tuple(found) < _ver_tuple(minimum):
        return Gate(f"version:{name}", False, f"{found}<{minimum}", mandatory=mandatory)
    return Gate(f"version:{name}", True, found, mandatory=mandatory)


def core_pin_check(found_version: Optional[str], pinned_minimum: str) -> Gate:
    """The shared runtime a kit imports must be at least the version the kit was built against."""
    if found_version is None:
        return Gate("core_pin", False, "core runtime not importable")
    if _ver_tuple(found_version) < _ver_tuple(pinned_minimum):
        return Gate("core_pin", False, f"core {found_version} older than pinned {pinned_minimum}")
    return Gate("core_pin", True, found_version)


# ----------------------------------------------------------------------------- digests
def sha256_file(path, chunk: int = 1 << 20) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(chunk)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def read_sums(path) -> Dict[str, str]:
    out = {}
    with open(path, "r", encoding="utf-8") as f:
        for ln in f:
            parts = ln.split()
            if len(parts) >= 2 and len(parts[0]) == 64:
                out[parts[-1].lstrip("*")] = parts[0]
    return out


def sums_gate(sums_path, root=None, name: str = "carry") -> Gate:
    """Every file listed in a ``SHA256SUMS`` exists under ``root`` with the listed digest."""
    root = root or os.path.dirname(os.path.abspath(sums_path))
    try:
        sums = read_sums(sums_path)
    except OSError as e:
        return Gate(name, False, f"cannot read {sums_path}: {e}")
    bad = []
    for rel, want in sums.items():
        p = os.path.join(root, rel)
        if not os.path.exists(p):
            bad.append(f"{rel}:missing")
        elif sha256_file(p) != want:
            bad.append(f"{rel}:digest")
    return Gate(name, not bad, ",".join(bad[:4]) + ("..." if len(bad) > 4 else "") if bad else f"{len(sums)}files")


def binary_refusal(path, expected_sha256: Optional[str]) -> Optional[str]:
    """Reason not to load a prebuilt binary (``.so`` / cubin), or None when it may be loaded: it must
    exist and, when a digest is recorded, match it byte for byte."""
    if not os.path.exists(path):
        return f"binary_missing:{os.path.basename(path)}"
    if expected_sha256 and sha256_file(path) != expected_sha256:
        return f"binary_digest_mismatch:{os.path.basename(path)}"
    return None
