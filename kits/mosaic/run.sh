#!/bin/bash
# mosaic kit (mosaic / joltz) on the B200-native framework - single entry point.
#   run.sh install [--weights DIR]      build the sm_100a kernel library, check the installation
#   run.sh check   [--config b200] [--mode M] [--n_gpu P]   dry run: resolve the mode, run the gates, print what would engage
#   run.sh design [--config b200] [--mode off|exact|fast|big] [--allow-partial] [--det 1] ...
# Mode = --mode when given, else MOSAIC_OPT from the environment, else the kit default (fast).
# Every run prints one "[mosaic-opt] ACTIVE mode=..." line; a mode that cannot engage prints
# "[mosaic-opt] NOT ACTIVE: <reason>" and exits 3 - never a silent fallback.
# Exit codes: 0 ok, 1 failed / outputs short, 2 usage, 3 not active or partial activation.
set -euo pipefail
HERE=$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)
ROOT=$(cd "$HERE/../.." && pwd)
export MODEL_OPT=$HERE
export PYTHONPATH="$ROOT${PYTHONPATH:+:$PYTHONPATH}"
[ $# -ge 1 ] || { sed -n '2,10p' "$0" >&2; exit 2; }
exec python -m uplifting_biomolecular_modeling_b200.kits mosaic "$@"
