"""Kit runtime: resolve the mode, run the gates, apply the mode's levers, speak the line protocol.

``Activation`` is what ``enable()`` and the CLI share: it prints exactly one ``ACTIVE`` line (or one
``NOT ACTIVE`` line and the caller exits 3), one ``LEVER`` line per lever, registers the ``EXIT``
tally, and can write ``opt_manifest.json``.  Reference contract: README.md:24-50 of the reference,
boltz2/opt/boltz2_opt/__init__.py:1-20, report.py:3-15.
"""
from __future__ import annotations

import os
import sys
from typing import Dict, List, Mapping, Optional

from ..core import cell_census, counters, gates, manifest, modes, report
from . import levers as _levers
from .registry import KitSpec, get


class ActivationError(RuntimeError):
    pass


def mode_table(spec: KitSpec) -> modes.ModeTable:
    bases = {}
    if "fast" in spec.modes and "exact" in spec.modes:
        bases["fast"] = "exact"
    if "big" in spec.modes:
        bases["big"] = "fast" if "fast" in spec.modes else "exact"
    return modes.ModeTable(spec.name, {m: spec.levers.get(m, ()) for m in spec.modes}, spec.default, bases)


class Activation:
    def __init__(self, spec: KitSpec, mode: str, source: str = "cli", n_gpu: int = 1, strict: bool = True,
                 environ: Optional[Mapping[str, str]] = None, probe=None):
        self.spec, self.mode, self.source, self.n_gpu, self.strict = spec, mode, source, n_gpu, strict
        self.environ = os.environ if environ is None else environ
        self.table = mode_table(spec)
        self.levers_on: List[str] = []
        self.levers_off: Dict[str, str] = {}
        self.levers_skipped: Dict[str, str] = {}
        self.levers_dropped: Dict[str, str] = {}     # droppable levers that declined: reported, never PARTIAL
        self.evidence: Dict[str, dict] = {}
        self.words: List[str] = []
        self.gates: List[gates.Gate] = []
        self.probe = probe or gates.probe_gpus
        self.lines: List[str] = []

    # ------------------------------------------------------------------ helpers
    def _emit(self, text: str) -> None:
        self.lines.append(text)
        report.emit(text)

    def refuse(self, reason: str) -> "ActivationError":
        self._emit(report.not_active_line(self.spec.tag, reason, f"mode={self.mode} n_gpu={self.n_gpu}"))
        return ActivationError(reason)

    # ------------------------------------------------------------------ plan
    def plan(self) -> List[str]:
        """Gates and the lever list of the mode; raises ActivationError (after the NOT ACTIVE line)."""
        if self.mode not in self.table:
            raise self.refuse(f"unknown mode {self.mode!r}; known: {', '.join(self.table.names())}")
        if self.n_gpu not in self.spec.n_gpu:
            raise self.refuse(f"--n_gpu {self.n_gpu} is not offered by this kit (offered: "
                              f"{','.join(map(str, self.spec.n_gpu))})")
        if self.n_gpu > 1 and self.spec.family == "evo2":
            # the sequence kit's multi-GPU form is tensor parallelism, a lever of its fast mode
            if "tp_fused" not in self.table.levers(self.mode):
                raise self.refuse("--n_gpu > 1 is a fast-mode feature of this kit (tensor parallelism reorders sums)")
        elif self.n_gpu > 1 and self.mode != "big":
            raise self.refuse("--n_gpu > 1 is a big-mode feature (tile extents reorder sums)")
        names = list(self.table.levers(self.mode))
        if self.n_gpu == 1 and "rowpair_tp" in names:
            names.remove("rowpair_tp")
        needs_gpu = any(_levers.LEVERS[n].needs_gpu for n in names if n in _levers.LEVERS)
        if needs_gpu:
            ok, gs = gates.run_gates([lambda: gates.gpu_gate(100, self.environ.get("MODEL_OPT_TARGET_GPU"),
                                                              self.probe, self.n_gpu)])
            self.gates = gs
            bad = gates.first_failure(gs)
            if bad is not None:
                raise self.refuse(f"gate {bad.name}: {bad.detail}")
            self.words = report.collect_words(gs)
        off = set(modes.levers_off(self.environ))
        plan = []
        for n in names:
            if n in off:
                self.levers_off[n] = "user"
            else:
                plan.append(n)
        return plan

    # ------------------------------------------------------------------ apply
    def apply(self, predictor=None, dry_run: bool = False) -> "Activation":
        plan = self.plan()
        for n in plan:
            lv = _levers.LEVERS.get(n)
            if lv is None:
                self.levers_skipped[n] = "unknown_lever"
                continue
            if dry_run or predictor is None or lv.apply is None:
                self.levers_on.append(n)
                continue
            try:
                if hasattr(predictor, "__dict__") and not hasattr(predictor, "n_gpu"):
                    predictor.n_gpu = self.n_gpu
                self.evidence[n] = lv.apply(predictor) or {}
                self.levers_on.append(n)
            except BaseException as e:  # noqa: BLE001
                why = f"{type(e).__name__}:{report.token(str(e))[:80]}"
                if lv.droppable:
                    self.levers_dropped[n] = why
                elif gates.is_cannot_run(e):
                    raise self.refuse(f"lever {n} cannot run: {e}")
                else:
                    self.levers_skipped[n] = why
        verb = "DRY-RUN" if dry_run else "ACTIVE"
        self._emit(report.with_words(report.line(self.spec.tag, verb, ("mode", self.mode),
                                                 ("levers", self.levers_on or None), ("source", self.source),
                                                 ("n_gpu", self.n_gpu)), self.words))
        for n in list(self.table.levers(self.mode)):
            lv = _levers.LEVERS.get(n)
            impl = lv.impl if lv else "unknown"
            strat = lv.strategy if lv else None
            origin = lv.origin if lv else "kit"
            if n in self.levers_on:
                self._emit(report.lever_line(self.spec.tag, n, "on", impl=impl, origin=origin, strategy=strat))
            elif n in self.levers_off:
                self._emit(report.lever_line(self.spec.tag, n, "off", reason=self.levers_off[n], impl=impl,
                                             origin=origin, strategy=strat))
            elif n in self.levers_skipped or n in self.levers_dropped:
                why = self.levers_skipped.get(n) or self.levers_dropped.get(n)
                self._emit(report.lever_line(self.spec.tag, n, "skipped", reason=why, impl=impl,
                                             origin=origin, strategy=strat))
        return self

    # ------------------------------------------------------------------ exit
    def report_dict(self) -> dict:
        partial = dict(self.levers_skipped)
        partial.update(counters.BOOK.partial())
        return {"partial": sorted(partial), "reasons": partial, "words": self.words}

    def finish(self, rc: int, allow_partial: bool = False, out_dir: Optional[str] = None,
               incomplete: Optional[str] = None) -> int:
        rep = self.report_dict()
        v = report.verdict(rc, rep, allow_partial, incomplete)
        pl = report.partial_line(self.spec.tag, v, rep["reasons"])
        if pl:
            self._emit(pl)
        if out_dir:
            manifest.write(out_dir, manifest.build(self.spec.name, self.mode, self.source, self.levers_on,
                                                   self.levers_skipped, self.words, v,
                                                   gpu=self.gates[0].detail if self.gates else None,
                                                   ledgers=counters.BOOK.stats(),
                                                   extra={"n_gpu": self.n_gpu, "levers_off": self.levers_off,
                                                          "levers_dropped": self.levers_dropped,
                                                          "lever_evidence": self.evidence,
                                                          **getattr(self, "manifest_extra", {})}))
        return v["exit_code"]

    def register_exit(self, rc_getter=lambda: 0) -> None:
        def line():
            stats = {"activation": {"mode": self.mode, "n_gpu": self.n_gpu, "active": True,
                                    "levers": len(self.levers_on)}}
            stats.update({k: v for k, v in counters.BOOK.stats().items()})
            return report.exit_line(self.spec.tag, " ".join(report.tally_fields(stats)), rc=rc_getter())
        report.register_exit_tally(self.spec.tag, line)
        cell_census.install_exit_report(self.spec.tag)


_ACTIVE: Dict[str, Activation] = {}


def enable(kit: str, mode: Optional[str] = None, strict: bool = True, trigger: Optional[str] = None,
           environ: Optional[Mapping[str, str]] = None, probe=None) -> Activation:
    """Library-style activation (``<KIT>_OPT=<mode>`` or an ``enable()`` call in the user's script).
    Models built afterwards through :func:`predictor` run under the mode.  Raises on refusal after
    printing NOT ACTIVE (the autoload hook turns that into exit 3)."""
    spec = get(kit)
    env = os.environ if environ is None else environ
    res = modes.resolve_mode(mode_table(spec), mode, spec.env, env)
    act = Activation(spec, res.mode, res.source, 1, strict, env, probe)
    if res.mode == "off":
        return act
    act.apply(None, dry_run=False)
    _ACTIVE[kit] = act
    act.register_exit()
    return act


def predictor(kit: str, config: Optional[str] = None, device: Optional[str] = None, **kw):
    """A :class:`~..api.Predictor` for a cofolding kit under the kit's active mode (``enable`` or ``<KIT>_OPT``): the
    model is built on its plain statements and the mode's levers are applied to it one by one.  Without an active
    mode the predictor runs ``off``."""
    import torch
    from .. import api
    spec = get(kit)
    act = _ACTIVE.get(kit)
    dev = device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    pred = api.Predictor(config or spec.config, mode="off", device=dev,
                         dtype=torch.bfloat16 if dev != "cpu" else torch.float32, **kw)
    if act is not None and act.mode != "off":
        pred.set_mode(act.mode)
        applied = Activation(spec, act.mode, act.source, 1, act.strict, act.environ, act.probe)
        applied.apply(pred)
        _ACTIVE[kit] = applied
    return pred


def status(kit: str) -> dict:
    act = _ACTIVE.get(kit)
    if act is None:
        return {"kit": kit, "active": False, "mode": "off"}
    return {"kit": kit, "active": True, "mode": act.mode, "levers": list(act.levers_on), "words": list(act.words)}
