"""Command line of a kit: ``python -m uplifting_biomolecular_modeling_b200.kits <kit> <verb> [options]``.

Verbs: ``install`` (build the kernel library, check the installation), ``check`` (dry run: resolve
the mode, run the gates, print what would engage), and the kit's run commands (``pred`` for the
cofolding kits; ``score`` / ``generate`` for the language models; ``design``; ``predict``).
``--mode off|exact|fast|big`` (CLI > ``<KIT>_OPT`` > kit default), ``--n_gpu P`` (big mode),
``--allow-partial``, ``--det 1``.  Exit codes 0 / 1 / 2 / 3 as in :mod:`core.report`.
Reference: <kit>/run.sh and <kit>/opt/<kit>_opt/cli.py of every reference kit.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import List, Optional

from ..core import det, modes, report
from . import base
from .registry import REGISTRY, get


def _parser(kit: str) -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog=f"{kit}", add_help=True)
    ap.add_argument("verb")
    ap.add_argument("--mode", default=None)
    ap.add_argument("--config", default="b200", help="card configuration (configs/<card>.env)")
    ap.add_argument("--n_gpu", type=int, default=1)
    ap.add_argument("--allow-partial", action="store_true")
    ap.add_argument("--det", type=int, default=0)
    ap.add_argument("--input", default=None)
    ap.add_argument("--out_dir", default=None)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--tokens", type=int, default=None, help="synthetic input: number of tokens")
    ap.add_argument("--msa_depth", type=int, default=None)
    ap.add_argument("--recycling_steps", type=int, default=None)
    ap.add_argument("--sampling_steps", type=int, default=None)
    ap.add_argument("--diffusion_samples", type=int, default=None)
    ap.add_argument("--weights", default=None)
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--model_config", default=None, help="override the kit's model configuration key")
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--max_new_tokens", type=int, default=32)
    ap.add_argument("--specdec", type=int, default=0,
                    help="evo2 generate: k > 0 decodes speculatively with k proposals per round from a draft model")
    ap.add_argument("--pth-dir", dest="pth_dir", default=None,
                    help="install: site directory that receives <kit>_opt_autoload.pth (in-process activation by "
                         "<KIT>_OPT=<mode>)")
    ap.add_argument("--upstream-fix", dest="upstream_fix", default=None,
                    help="comma-separated corrections to the stock model that change outputs on purpose")
    return ap


def main(argv: Optional[List[str]] = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help"):
        print("usage: kits <kit> <verb> [--mode M] [--n_gpu P] ...; kits: " + ", ".join(sorted(REGISTRY)),
              file=sys.stderr)
        return report.EXIT_USAGE
    kit = argv[0]
    try:
        spec = get(kit)
    except KeyError as e:
        print(str(e), file=sys.stderr)
        return report.EXIT_USAGE
    try:
        args = _parser(kit).parse_args(argv[1:])
    except SystemExit:
        return report.EXIT_USAGE
    if args.verb not in spec.commands:
        print(f"{kit}: unknown verb {args.verb!r}; verbs: {', '.join(spec.commands)}", file=sys.stderr)
        return report.EXIT_USAGE
    # card configuration
    from ..core import home
    cfgp = home.config_path(kit, args.config)
    if cfgp:
        modes.EnvScript.from_file(cfgp).apply()
    undeclared = modes.check_declared_env(spec.env, [spec.env, spec.env + "_ALLOW_PARTIAL"])
    if undeclared:
        report.emit(report.not_active_line(spec.tag, f"undeclared variable(s) {','.join(undeclared)}"))
        return report.EXIT_NOT_ACTIVE
    if args.upstream_fix:
        from ..core import upstream_fix
        try:
            upstream_fix.resolve(upstream_fix.parse(args.upstream_fix), kit)
        except upstream_fix.UnknownFix as e:
            print(f"{kit}: {e}", file=sys.stderr)
            return report.EXIT_USAGE
    if args.verb == "install":
        return _install(spec, args)
    try:
        res = modes.resolve_mode(base.mode_table(spec), args.mode, spec.env)
    except modes.ModeError as e:
        report.emit(report.not_active_line(spec.tag, str(e)))
        return report.EXIT_NOT_ACTIVE
    if args.det:
        det.apply_env(det.Recipe(seed=args.seed))
    act = base.Activation(spec, res.mode, res.source, args.n_gpu)
    allow = report.allow_partial(args.allow_partial, spec.env + "_ALLOW_PARTIAL")
    if args.verb == "check":
        try:
            act.apply(None, dry_run=True)
        except base.ActivationError:
            return report.EXIT_NOT_ACTIVE
        return act.finish(0, allow)
    from . import run as _run
    return _run.run(spec, act, args, allow)


def _install(spec, args) -> int:
    from ..ops import build
    try:
        path = build.build()
    except Exception as e:  # noqa: BLE001
        report.emit(report.line(spec.tag, "INSTALL", ("state", "failed"), ("reason", report.token(str(e))[:160])))
        return report.EXIT_FAIL
    pth = None
    if args.pth_dir:
        from . import autoload_hook
        try:
            pth = autoload_hook.place_pth(spec.name, args.pth_dir)
        except OSError as e:
            report.emit(report.line(spec.tag, "INSTALL", ("state", "failed"), ("reason", report.token(str(e))[:160])))
            return report.EXIT_FAIL
    report.emit(report.line(spec.tag, "INSTALL", ("state", "ok"), ("library", path), ("weights", args.weights),
                            ("pth", pth)))
    if args.weights:
        os.makedirs(args.weights, exist_ok=True)
    return report.EXIT_OK


if __name__ == "__main__":
    sys.exit(main())
