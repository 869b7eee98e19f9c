"""Child processes: logged runs under a process-group watchdog, step runners, clean child environments.

``run_logged`` starts a command in its own process group, tees its output to a log, and on timeout
(or when the parent is interrupted) terminates the whole group: SIGTERM, a grace period, SIGKILL.
Only the group this function started is ever signalled.  Reference: common/opt_core/opt_core/process.py:52,94,109.
"""
from __future__ import annotations

import os
import signal
import subprocess
import sys
import time
from typing import Mapping, Optional, Sequence

KILL_GRACE_S = 10.0


def child_env(base: Optional[Mapping[str, str]] = None, drop_prefixes: Sequence[str] = (),
              extra: Optional[Mapping[str, str]] = None) -> dict:
    """Copy of the environment without variables of the given prefixes (a stock child must not
    inherit a kit's variables), plus ``extra``."""
    env = dict(os.environ if base is None else base)
    for k in list(env):
        if any(k.startswith(p) for p in drop_prefixes):
            del env[k]
    if extra:
        env.update({k: str(v) for k, v in extra.items()})
    return env


def _terminate_group(proc: subprocess.Popen, grace: float) -> None:
    try:
        pgid = os.getpgid(proc.pid)
    except (ProcessLookupError, PermissionError):
        return
    for sig, wait in ((signal.SIGTERM, grace), (signal.SIGKILL, 2.0)):
        try:
            os.killpg(pgid, sig)
        except (ProcessLookupError, PermissionError):
            return
        t0 = time.time()
        while time.time() - t0 < wait:
            if proc.poll() is not None:
                return
            time.sleep(0.05)


def run_logged(cmd: Sequence[str], log_path: Optional[str] = None, env: Optional[Mapping[str, str]] = None,
               timeout_s: Optional[float] = None, cwd: Optional[str] = None, echo: bool = False,
               grace_s: float = KILL_GRACE_S) -> int:
    """Run ``cmd`` in a new process group; returns its exit code, or 124 on timeout."""
    log = open(log_path, "ab") if log_path else None
    try:
        proc = subprocess.Popen(list(cmd), stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env, cwd=cwd,
                                start_new_session=True)
        t0 = time.time()
        assert proc.stdout is not None
        os.set_blocking(proc.stdout.fileno(), False)
        while True:
            chunk = proc.stdout.read()
            if chunk:
                if log:
                    log.write(chunk)
                    log.flush()
                if echo:
                    sys.stderr.buffer.write(chunk)
                    sys.stderr.flush()
            if proc.poll() is not None:
                rest = proc.stdout.read()
                if rest:
                    if log:
                        log.write(rest)
                    if echo:
                        sys.stderr.buffer.write(rest)
                return proc.returncode
            if timeout_s is not None and time.time() - t0 > timeout_s:
                _terminate_group(proc, grace_s)
                return 124
            time.sleep(0.02)
    except KeyboardInterrupt:
        _terminate_group(proc, grace_s)
        raise
    finally:
        if log:
            log.close()


def run_step(name: str, cmd: Sequence[str], tag: str = "opt_core", **kw) -> int:
    """``run_logged`` with STEP / DONE lines around it."""
    from . import report
    report.emit(report.line(tag, "STEP", ("name", name), ("cmd", report.token(" ".join(cmd))[:120])))
    t0 = time.time()
    rc = run_logged(cmd, **kw)
    report.emit(report.line(tag, "DONE", ("name", name), ("rc", rc), ("seconds", round(time.time() - t0, 2))))
    return rc
