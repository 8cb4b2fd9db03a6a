#!/usr/bin/env bash
# Launch pretraining on every GPU of this node (one process per GPU).
#
#   ./scripts/train.sh <config.yaml> [--resume DIR] [--auto_resume] [--max_checkpoints N] ...
#   NPROC=2 ./scripts/train.sh configs/bench/xs_standard.yaml --max_steps 20
#   DEVICE=cpu NPROC=2 ./scripts/train.sh configs/bench/tiny_cpu.yaml      # gloo, no GPU needed
#   ./scripts/train.sh configs/scaling/l_standard.yaml --parallel_mode fsdp  # ddp | zero | fsdp (default: config / zero)
#
# Everything after the config path is passed to train.py unchanged.
set -euo pipefail
cd "$(dirname "$0")/.."

if [[ -f .env ]]; then set -a; source .env; set +a; fi

if [[ $# -lt 1 ]]; then
  echo "Usage: $0 <config> [train.py flags]"; echo; echo "Available configs:"; find configs -name '*.yaml' | sort
  exit 1
fi
CONFIG="$1"; shift
[[ -f "$CONFIG" ]] || { echo "ERROR: config not found: $CONFIG"; exit 1; }

DEVICE="${DEVICE:-cuda}"
if [[ -z "${NPROC:-}" ]]; then
  if [[ "$DEVICE" == "cuda" ]]; then NPROC="$(python -c 'import torch; print(max(1, torch.cuda.device_count()))')"; else NPROC=1; fi
fi
PORT="${MASTER_PORT:-29500}"

echo "========================================"
echo "  Config : $CONFIG"
echo "  Procs  : $NPROC ($DEVICE)"
echo "  Extra  : ${*:-none}"
echo "========================================"

# NVLink SHARP reductions on NVSwitch systems; one work queue per device keeps kernel order = launch order.
export NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-1}"
export CUDA_DEVICE_MAX_CONNECTIONS="${CUDA_DEVICE_MAX_CONNECTIONS:-1}"

exec python -m torch.distributed.run --nnodes="${NNODES:-1}" --node-rank="${NODE_RANK:-0}" \
  --nproc-per-node "$NPROC" --master-addr "${MASTER_ADDR:-127.0.0.1}" --master-port "$PORT" \
  train.py --config "$CONFIG" --device "$DEVICE" "$@"
