"""Generate the per-kit entry points: ``kits/<kit>/run.sh``, ``configs/b200.env``, ``CHANGES.md`` (what each mode
changes, lever by lever) and the ``.pth`` hook
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
NCCL_NVLS_ENABLE=${{NCCL_NVLS_ENABLE:-0}}
"""


FAMILY_MODULE = {
    "cofold": "models/cofold.py (Pairformer trunk, MSA module, template embedder, diffusion sampler, confidence head)",
    "design": "models/cofold.py structure trunk with the design conditioning levers; models/design.py (sequence inversion, inverse-folding decoder) for ef2inv / proteinmpnn / esm_if1",
    "evo2": "models/evo2.py (StripedHyena-2; tensor parallel through parallel/tp.py)",
    "protein_lm": "models/plm.py (ESM-C / E1 / ProGen2 / GPN-Star block forms)",
    "genomic_track": "models/genomics.py (Enformer / Borzoi / Flashzoi / ChromBPNet)",
}

CHANGES = """# {name} - what each mode changes

Upstream: {upstream}.  Served by `{module}`.
Entry point: `kits/{name}/run.sh` (verbs: {verbs}); library use: `{env}=<mode>` or
`uplifting_biomolecular_modeling_b200.kits.base.enable("{name}", mode)`.{library}

| mode | meaning |
|---|---|
| `off` | the plain PyTorch statements, nothing engaged; the process is proven clean of kit state (`STOCK clean=True`) |
{mode_rows}

GPUs per run: {ngpu}.{ceiling}

## Levers by mode

{lever_tables}

Every lever prints one `[{tag}] LEVER name=... state=engaged|skipped reason=...` line and is counted in the run's
ledger; `MODEL_OPT_LEVERS_OFF=<lever,...>` removes levers from a mode (the run then reports a partial activation
and exits 3 unless `--allow-partial`).  A mode that cannot engage prints `[{tag}] NOT ACTIVE: <reason>` and exits 3;
kernels that fail their load-time check against the fp32 statements exit 5 (`KERNELS-REFUSED`).
"""

MODE_MEANING = {
    "exact": "| `exact` | the same statements with the sampler / forward step (and small Pairformer stacks) replayed from CUDA graphs whose first replay is checked bit for bit against eager; outputs bitwise equal to `off` |",
    "fast": "| `fast` | the sm_100a kernel path in bf16 (tcgen05 kernels, fused row kernels, CUDA graphs); outputs within the documented tolerance of `off`; every module call is counted served / fallback and an undeclared fallback ends the run PARTIAL (exit 3) |",
    "big": "| `big` | `fast` plus the memory levers (pair operations in row blocks, trunk scratch released before the sampler, initial pair tensor parked in pinned host memory, expandable allocator segments) and, with `--n_gpu P`, the row-sharded pair tensor over peer memory; rank 0 runs sampler and confidence head and writes coordinates |",
}


def changes_text(spec) -> str:
    from .levers import LEVERS
    tables = []
    for mode in spec.modes:
        names = spec.levers.get(mode, ())
        if not names:
            continue
        def what(n):
            doc = (LEVERS[n].apply.__doc__ or "").strip().split("\n\n")[0] if LEVERS[n].apply else ""
            return " ".join(doc.split()) or "switches the named modules to their kernel implementation"
        rows = "\n".join(f"| `{n}` | {LEVERS[n].strategy} | `{LEVERS[n].impl}` | {'yes' if LEVERS[n].needs_gpu else 'no'} | "
                         f"{what(n)} |" for n in names if n in LEVERS)
        tables.append(f"### `{mode}`\n\n| lever | strategy | implemented by | needs a GPU | what it does |\n"
                      f"|---|---|---|---|---|\n{rows}")
    return CHANGES.format(
        name=spec.name, upstream=spec.upstream, module=FAMILY_MODULE.get(spec.family, spec.family),
        verbs=", ".join(spec.commands), env=spec.env, tag=spec.tag,
        library=("  Library-style kit: no mode is on by default; name one." if spec.library_style else
                 f"  Default mode: `{spec.default}`."),
        mode_rows="\n".join(MODE_MEANING[m] for m in spec.modes if m in MODE_MEANING),
        ngpu=", ".join(str(n) for n in spec.n_gpu),
        ceiling=("" if not spec.big_token_ceiling else
                 f"  The reference states a single-GPU `big` ceiling of {spec.big_token_ceiling} tokens on an 80 GB card."),
        lever_tables="\n\n".join(tables) or "(no levers beyond the mode's definition)")


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
        with open(os.path.join(d, "CHANGES.md"), "w") as f:
            f.write(changes_text(spec))
        n += 1
    return n


if __name__ == "__main__":
    print(f"generated {generate()} kits under {home.kits_root()}")
