"""Launcher of a row-sharded run: one worker process per GPU, fail-fast teardown, bounded waits.

The parent spawns P workers with ``ROWPAIR_{RANK,WORLD,LOCAL_RANK,ADDR,PORT}`` (and one
``PYTHONHASHSEED`` for all of them), polls them, and on the first non-zero exit terminates the rest
(SIGTERM, then SIGKILL after a grace period) and raises :class:`RankFailed` with the failing rank's log
tail.  Only processes this launcher started are ever signalled, by their exact pids.  Workers call
:func:`init_from_env` to join the group (NCCL on GPUs, gloo on CPU) with a bounded collective timeout so
that a dead peer surfaces as an error, and register an exit guard that prints ``RANKSTUCK`` and leaves
with ``os._exit`` if teardown blocks.  Reference: common/opt_core/opt_core/mem/rowpair/launch.py:28-31,
80,88,163,367,493,515 and dist.py:946,1106-1212.
"""
from __future__ import annotations

import datetime
import os
import signal
import socket
import subprocess
import sys
import tempfile
import threading
import time
from typing import Callable, Dict, List, Mapping, Optional, Sequence

from ..core import report

KILL_GRACE_S = 10.0
FAIL_GRACE_S = 60.0
TAG = "rowpair"


class RankFailed(RuntimeError):
    def __init__(self, rank: int, rc: int, tail: str):
        super().__init__(f"rank {rank} exited with code {rc}\n{tail}")
        self.rank, self.rc, self.tail = rank, rc, tail


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def rank_env(rank: int, world: int, port: int, base: Optional[Mapping[str, str]] = None, cpu: bool = False,
             extra: Optional[Mapping[str, str]] = None) -> Dict[str, str]:
    env = dict(os.environ if base is None else base)
    env.update({"ROWPAIR_RANK": str(rank), "ROWPAIR_WORLD": str(world), "ROWPAIR_LOCAL_RANK": str(rank),
                "ROWPAIR_ADDR": "127.0.0.1", "ROWPAIR_PORT": str(port),
                "RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port),
                "PYTHONHASHSEED": env.get("PYTHONHASHSEED", "0")})
    if cpu:
        env["ROWPAIR_BACKEND"] = "gloo"
    else:
        # A rank that leaves (or is stopped by the fail-fast teardown) must hold no NVLink multicast binding: the
        # package's kernels use plain peer loads and stores, so nothing is lost by keeping multicast off in NCCL and
        # in torch's symmetric memory for rank processes.  A caller that wants NVLS sets the variables itself.
        env.setdefault("NCCL_NVLS_ENABLE", "0")
        env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if extra:
        env.update({k: str(v) for k, v in extra.items()})
    return env


def rankenv_line(rank: int, env: Mapping[str, str]) -> str:
    keys = ("ROWPAIR_RANK", "ROWPAIR_WORLD", "ROWPAIR_PORT", "PYTHONHASHSEED")
    return report.line(TAG, "RANKENV", *[(k.lower(), env.get(k)) for k in keys])


def _tail(path: str, n: int = 30) -> str:
    try:
        with open(path, "r", errors="replace") as f:
            return "".join(f.readlines()[-n:])
    except OSError:
        return ""


def _stop(procs: Sequence[subprocess.Popen], grace_s: float) -> None:
    for p in procs:
        if p.poll() is None:
            try:
                p.send_signal(signal.SIGTERM)
            except ProcessLookupError:
                pass
    t0 = time.time()
    while time.time() - t0 < grace_s and any(p.poll() is None for p in procs):
        time.sleep(0.05)
    for p in procs:
        if p.poll() is None:
            try:
                p.kill()
            except ProcessLookupError:
                pass


def run_rank_processes(world: int, argv: Sequence[str], cpu: bool = False, run_timeout_s: float = 3600.0,
                       kill_grace_s: float = KILL_GRACE_S, log_dir: Optional[str] = None,
                       extra_env: Optional[Mapping[str, str]] = None, echo_rank0: bool = True) -> List[int]:
    """Run ``argv`` as ``world`` rank processes.  Returns the exit codes (all zero) or raises RankFailed."""
    port = free_port()
    log_dir = log_dir or tempfile.mkdtemp(prefix="rowpair_logs_")
    os.makedirs(log_dir, exist_ok=True)
    procs: List[subprocess.Popen] = []
    logs: List[str] = []
    try:
        for r in range(world):
            env = rank_env(r, world, port, cpu=cpu, extra=extra_env)
            lp = os.path.join(log_dir, f"rank{r}.log")
            logs.append(lp)
            f = open(lp, "wb")
            procs.append(subprocess.Popen(list(argv), env=env, stdout=f, stderr=subprocess.STDOUT))
            f.close()
        t0 = time.time()
        while True:
            codes = [p.poll() for p in procs]
            bad = [(r, c) for r, c in enumerate(codes) if c not in (None, 0)]
            if bad:
                r, c = bad[0]
                _stop(procs, kill_grace_s)
                report.emit(report.line(TAG, "RANKEXIT", ("rank", r), ("rc", c)))
                raise RankFailed(r, c, _tail(logs[r]))
            if all(c == 0 for c in codes):
                break
            if time.time() - t0 > run_timeout_s:
                _stop(procs, kill_grace_s)
                stuck = [r for r, c in enumerate(codes) if c is None]
                raise RankFailed(stuck[0], 124, f"run timed out after {run_timeout_s}s; stuck ranks {stuck}\n"
                                 + _tail(logs[stuck[0]]))
            time.sleep(0.05)
        if echo_rank0:
            sys.stderr.write(_tail(logs[0], 200))
        return [0] * world
    finally:
        _stop(procs, 0.0)


def run_sharded(world: int, entry: str, args: Sequence[str] = (), cpu_ok: bool = False, backend: Optional[str] = None,
                **kw) -> List[int]:
    """Run ``python -m <entry> <args>`` as ``world`` ranks."""
    cpu = bool(cpu_ok and (backend == "gloo"))
    return run_rank_processes(world, [sys.executable, "-m", entry, *args], cpu=cpu, **kw)


# ----------------------------------------------------------------------------- worker side
_EXIT_GUARD = {"armed": False}


def init_from_env(timeout_s: Optional[float] = None):
    """Join the process group described by ROWPAIR_* / torchrun variables; returns a GroupComm."""
    import torch
    import torch.distributed as dist
    from .comm import GroupComm
    rank = int(os.environ.get("ROWPAIR_RANK", os.environ.get("RANK", "0")))
    world = int(os.environ.get("ROWPAIR_WORLD", os.environ.get("WORLD_SIZE", "1")))
    local = int(os.environ.get("ROWPAIR_LOCAL_RANK", os.environ.get("LOCAL_RANK", "0")))
    addr = os.environ.get("ROWPAIR_ADDR", os.environ.get("MASTER_ADDR", "127.0.0.1"))
    port = os.environ.get("ROWPAIR_PORT", os.environ.get("MASTER_PORT", "29500"))
    backend = os.environ.get("ROWPAIR_BACKEND") or ("nccl" if torch.cuda.is_available() else "gloo")
    timeout_s = float(os.environ.get("ROWPAIR_NCCL_TIMEOUT_S", timeout_s or 1800))
    kw = {}
    if backend == "nccl":
        torch.cuda.set_device(local)
        kw["device_id"] = torch.device("cuda", local)
    dist.init_process_group(backend, init_method=f"tcp://{addr}:{port}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=timeout_s), **kw)
    store = None
    try:
        store = dist.distributed_c10d._get_default_store()
    except Exception:  # noqa: BLE001
        pass
    arm_exit_guard(rank)
    return GroupComm(store=store)


def arm_exit_guard(rank: int, grace_s: Optional[float] = None) -> None:
    """If interpreter exit (group teardown) blocks for longer than the grace, print RANKSTUCK and leave."""
    import atexit
    if _EXIT_GUARD["armed"]:
        return
    _EXIT_GUARD["armed"] = True
    grace = float(os.environ.get("ROWPAIR_EXIT_GRACE_S", grace_s or 90))

    def guard():
        def stuck():
            report.emit(report.line(TAG, "RANKSTUCK", ("rank", rank), ("grace_s", grace)))
            report.forced_exit(70)
        t = threading.Timer(grace, stuck)
        t.daemon = True
        t.start()
        try:
            import torch.distributed as dist
            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
        t.cancel()
        report.emit(report.line(TAG, "RANKLEAVE", ("rank", rank)))

    atexit.register(guard)


def run_prediction_sharded(spec, act, args, config: str, allow_partial: bool) -> int:
    """``pred --mode big --n_gpu P``: start P ranks of ``parallel.worker``; the parent prints ACTIVE and EXIT."""
    act.levers_on = act.plan()
    ckpt = args.checkpoint or args.weights
    if ckpt:
        # names and shapes are held against a model on the meta device before any rank starts, so that a checkpoint
        # that does not fit is NOT ACTIVE with exit 3 instead of a failed rank
        import torch
        from ..models import cofold, mappers, weights
        try:
            with torch.device("meta"):
                probe = cofold.CofoldModel(cofold.CONFIGS[config])
            rep = weights.load_checkpoint(probe, ckpt, strict=not allow_partial, dry_run=True,
                                          mapper=mappers.for_kit(spec.name))
        except (ValueError, OSError) as e:
            act.refuse(f"checkpoint {ckpt}: {e}")
            return report.EXIT_NOT_ACTIVE
        report.emit(report.line(spec.tag, "WEIGHTS", ("path", ckpt), ("matched", rep.matched),
                                ("missing", len(rep.missing)), ("unexpected", len(rep.unexpected)),
                                ("shape_mismatch", len(rep.shape_mismatch)), ("init_skipped", 0)))
    report.emit(report.with_words(report.line(spec.tag, "ACTIVE", ("mode", act.mode), ("levers", act.levers_on),
                                              ("source", act.source), ("n_gpu", act.n_gpu),
                                              ("sharding", "rowpair")), act.words))
    wargs = ["--config", config, "--tokens", str(args.tokens or 256), "--msa_depth", str(args.msa_depth or 1),
             "--seed", str(args.seed), "--structure", "1", "--kit", spec.name]
    if args.out_dir:
        wargs += ["--out_dir", args.out_dir]
    if args.recycling_steps is not None:
        wargs += ["--recycles", str(args.recycling_steps)]
    for flag, val in (("--input", args.input), ("--checkpoint", args.checkpoint or args.weights),
                      ("--sampling_steps", args.sampling_steps), ("--diffusion_samples", args.diffusion_samples)):
        if val is not None:
            wargs += [flag, str(val)]
    if allow_partial:
        wargs += ["--allow-partial"]
    try:
        run_sharded(act.n_gpu, "uplifting_biomolecular_modeling_b200.parallel.worker", wargs)
    except RankFailed as e:
        report.emit(report.line(spec.tag, "FAILED", ("rank", e.rank), ("rc", e.rc)))
        sys.stderr.write(e.tail)
        return act.finish(report.EXIT_FAIL, allow_partial, args.out_dir)
    return act.finish(0, allow_partial, args.out_dir)
