#!/bin/bash
# af3_jax kit (AlphaFold 3 (JAX fork)) on the B200-native framework - single entry point.
#   run.sh install [--weights DIR]      build the sm_100a kernel library, check the installation
#   run.sh check   [--config b200] [--mode M] [--n_gpu P]   dry run: resolve the mode, run the gates, print what would engage
#   run.sh pred [--config b200] [--mode off|exact|fast|big] [--n_gpu P] [--allow-partial] [--det 1] ...
# Mode = --mode when given, else AF3_JAX_OPT from the environment, else the kit default (fast).
# Every run prints one "[af3_jax-opt] ACTIVE mode=..." line; a mode that cannot engage prints
# "[af3_jax-opt] NOT ACTIVE: <reason>" and exits 3 - never a silent fallback.
# Exit codes: 0 ok, 1 failed / outputs short, 2 usage, 3 not active or partial activation.
set -euo pipefail
HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export MODEL_OPT=$HERE
export PYTHONPATH="$ROOT${PYTHONPATH:+:$PYTHONPATH}"
[ $# -ge 1 ] || { sed -n '2,10p' "$0" >&2; exit 2; }
exec python -m uplifting_biomolecular_modeling_b200.kits af3_jax "$@"
