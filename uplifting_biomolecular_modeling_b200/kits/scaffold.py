"""Generate the per-kit entry points: ``kits/<kit>/run.sh``, ``configs/b200.env`` and the ``.pth`` hook
package for library-style activation.  Run once after editing the registry:
``python -m uplifting_biomolecular_modeling_b200.kits.scaffold``.  The generated ``run.sh`` keeps the
reference's surface: ``run.sh install | check | <command> --config <card> --mode off|exact|fast|big
[--n_gpu P]`` (README.md:78-84 of the reference)."""
from __future__ import annotations

import os
import stat

from ..core import home
from .registry import REGISTRY

RUN_SH = """#!/bin/bash
# {name} kit ({upstream}) on the B200-native framework - single entry point.
#   run.sh install [--weights DIR]      build the sm_100a kernel library, check the installation
#   run.sh check   [--config b200] [--mode M] [--n_gpu P]   dry run: resolve the mode, run the gates, print what would engage
#   run.sh {cmds} [--config b200] [--mode {modes}]{ngpu} [--allow-partial] [--det 1] ...
# Mode = --mode when given, else {env} from the environment, else the kit default ({default}).
# Every run prints one "[{tag}] ACTIVE mode=..." line; a mode that cannot engage prints
# "[{tag}] NOT ACTIVE: <reason>" and exits 3 - never a silent fallback.
# Exit codes: 0 ok, 1 failed / outputs short, 2 usage, 3 not active or partial activation.
set -euo pipefail
HERE=$(cd "$(dirname "${{BASH_SOURCE[0]}}")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export MODEL_OPT=$HERE
export PYTHONPATH="$ROOT${{PYTHONPATH:+:$PYTHONPATH}}"
[ $# -ge 1 ] || {{ sed -n '2,10p' "$0" >&2; exit 2; }}
exec python -m uplifting_biomolecular_modeling_b200.kits {name} "$@"
"""

ENV = """# {name}: deployment parameters for an 8 x B200 (sm_100a, 180 GB HBM3e) host.  Sourced by run.sh --config b200.
# Only deployment parameters live here (target card, build-cache keying); the mode is never set here.
MODEL_OPT_TARGET_GPU=b200
MODEL_OPT_STACK_KEY=${{MODEL_OPT_STACK_KEY:-torch2.11-cu128-sm100a}}
MODEL_OPT_JIT_ROOT=${{MODEL_OPT_JIT_ROOT:-/tmp/model_opt_jit}}
NCCL_NVLS_ENABLE=${{NCCL_NVLS_ENABLE:-1}}
"""


def generate(root: str = None) -> int:
    root = root or home.kits_root()
    n = 0
    for name, spec in sorted(REGISTRY.items()):
        d = os.path.join(root, name)
        os.makedirs(os.path.join(d, "configs"), exist_ok=True)
        cmds = "|".join(c for c in spec.commands if c not in ("install", "check"))
        ngpu = " [--n_gpu P]" if len(spec.n_gpu) > 1 else ""
        p = os.path.join(d, "run.sh")
        with open(p, "w") as f:
            f.write(RUN_SH.format(name=name, upstream=spec.upstream, cmds=cmds, modes="|".join(spec.modes),
                                  ngpu=ngpu, env=spec.env, default=spec.default or "none: name one",
                                  tag=spec.tag))
        os.chmod(p, os.stat(p).st_mode | stat.S_IXUSR | stat.S_IXGRP | stat.S_IXOTH)
        with open(os.path.join(d, "configs", "b200.env"), "w") as f:
            f.write(ENV.format(name=name))
        n += 1
    return n


if __name__ == "__main__":
    print(f"generated {generate()} kits under {home.kits_root()}")
