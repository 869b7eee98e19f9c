"""K worker processes on one GPU (small models leave most of a B200 idle per process).

The workers are plain child processes sharing the device by time slicing.  If an MPS control daemon is already
running (``CUDA_MPS_PIPE_DIRECTORY`` set and its pipe present) they use it; this module never starts, stops or
configures a daemon - that is a property of the GPU its other users would inherit.  Each worker's log is scanned
with the shared OOM classifier: any worker that ran out of memory turns the result into exit code 6, so a caller
can retry with fewer workers.  Reference: common/mps_packing/mps_workers.sh:1-37.
"""
from __future__ import annotations

import os
import subprocess
from dataclasses import dataclass, field
from typing import List, Mapping, Optional, Sequence

from ..core import oom, report

EXIT_OOM = 6


@dataclass
class PackResult:
    returncodes: List[int] = field(default_factory=list)
    oom_workers: List[int] = field(default_factory=list)
    logs: List[str] = field(default_factory=list)

    @property
    def exit_code(self) -> int:
        if self.oom_workers:
            return EXIT_OOM
        return 0 if all(rc == 0 for rc in self.returncodes) else 1


def mps_available(environ: Optional[Mapping[str, str]] = None) -> bool:
    env = os.environ if environ is None else environ
    pipe = env.get("CUDA_MPS_PIPE_DIRECTORY")
    return bool(pipe) and os.path.exists(os.path.join(pipe, "control"))


def run_workers(commands: Sequence[Sequence[str]], log_dir: str, gpu: int = 0, tag: str = "opt_core",
                env: Optional[Mapping[str, str]] = None, timeout_s: Optional[float] = None) -> PackResult:
    """Run one command per worker concurrently on GPU ``gpu``; logs go to ``log_dir/worker_<i>.log``."""
    os.makedirs(log_dir, exist_ok=True)
    base = dict(os.environ if env is None else env)
    base["CUDA_VISIBLE_DEVICES"] = str(gpu)
    res = PackResult()
    procs = []
    for i, cmd in enumerate(commands):
        path = os.path.join(log_dir, f"worker_{i}.log")
        res.logs.append(path)
        f = open(path, "w")
        e = dict(base, UBM_WORKER_INDEX=str(i), UBM_WORKER_COUNT=str(len(commands)))
        procs.append((subprocess.Popen(list(cmd), stdout=f, stderr=subprocess.STDOUT, env=e), f))
    for i, (p, f) in enumerate(procs):
        try:
            rc = p.wait(timeout=timeout_s)
        except subprocess.TimeoutExpired:
            p.kill()                      # the exact child this function started
            rc = p.wait()
        f.close()
        res.returncodes.append(rc)
        with open(res.logs[i], errors="replace") as g:
            if oom.is_oom_text(g.read()):
                res.oom_workers.append(i)
    report.emit(report.line(tag, "PACK", ("workers", len(commands)), ("gpu", gpu), ("mps", mps_available(base)),
                            ("oom", len(res.oom_workers)), ("rc", res.exit_code)))
    return res
