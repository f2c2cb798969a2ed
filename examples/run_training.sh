#!/usr/bin/env bash
# End-to-end comparison on one node: this framework against the reference (when it is installed
# under baseline/_ref), same model shape, same number of steps.  Prints both step times.
set -euo pipefail
NGPU=${NGPU:-2}
STEPS=${STEPS:-10}
PORT=${PORT:-29517}
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
cd "$(dirname "$0")/.."
run() { python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 --master-port "$PORT" "$@"; }
echo "== fluidmoe_b200 =="
run bench.py --gpus "$NGPU" --steps "$STEPS" --warmup 3 | tail -1
echo "== reference =="
run bench.py --gpus "$NGPU" --steps "$STEPS" --warmup 3 --impl reference | tail -1
