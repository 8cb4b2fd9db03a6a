#!/usr/bin/env bash
# Run several experiment configs one after another on this node (each with auto-resume, so the
# script can simply be started again after an interruption).
#
#   ./scripts/launch_all.sh configs/scaling/xs_standard.yaml configs/scaling/xs_global.yaml
set -euo pipefail
cd "$(dirname "$0")/.."
[[ $# -ge 1 ]] || { echo "Usage: $0 <config> [<config> ...]"; exit 1; }
for cfg in "$@"; do
  echo ">>> $cfg"
  ./scripts/train.sh "$cfg" --auto_resume --max_checkpoints "${MAX_CHECKPOINTS:-3}"
done
