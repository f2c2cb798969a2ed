#!/usr/bin/env bash
# End-to-end comparison on one node, same model shape, same data, same number of steps:
#   1. this framework, overlapped (device-initiated transport where the GPUs reach each other,
#      scheduler in full mode);
#   2. this framework, baseline (library all-to-all, scheduler off);
#   3. the Megatron-Core arm and 4. the DeepSpeed arm, when those packages are installed;
#   5. the reference implementation (when installed under baseline/_ref): loss and gradient
#      parity of its layer stack against ours on identical weights (tools/parity_reference), which
#      is the form the reference's own driver validates itself in: final loss and gradient norm of
#      every arm side by side (examples/run_training.sh:243-290 of the reference).
# Every arm prints Megatron-format log lines; the table at the end shows the last step's loss,
# gradient norm and the median iteration time of each.
#   NGPU=8 STEPS=50 LAYERS=4 examples/run_training.sh [token_file]
set -uo pipefail
NGPU=${NGPU:-2}
STEPS=${STEPS:-20}
LAYERS=${LAYERS:-2}
HIDDEN=${HIDDEN:-1024}; HEADS=${HEADS:-8}; KV=${KV:-8}; FFN=${FFN:-2048}; EXPERTS=${EXPERTS:-8}; TOPK=${TOPK:-2}
SEQ=${SEQ:-2048}; VOCAB=${VOCAB:-32000}; LR=${LR:-3e-4}
PORT=${PORT:-29517}
DATA=${1:-${FLUIDMOE_DATASET_SOURCE:-}}
OUT=${OUT:-training_logs}
export CUDA_DEVICE_MAX_CONNECTIONS=${CUDA_DEVICE_MAX_CONNECTIONS:-1}
cd "$(dirname "$0")/.."
mkdir -p "$OUT"
SHAPE="--layers $LAYERS --hidden $HIDDEN --heads $HEADS --kv-heads $KV --ffn $FFN --experts $EXPERTS --top-k $TOPK \
  --seq $SEQ --vocab $VOCAB --lr $LR --steps $STEPS"
[ -n "$DATA" ] && SHAPE="$SHAPE --data $DATA"
launch() {  # launch <log> <script> [args]
  local log=$1; shift
  PORT=$((PORT + 1))
  if [ "$NGPU" -gt 1 ]; then
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NGPU" --master-addr 127.0.0.1 \
      --master-port "$PORT" "$@" > "$OUT/$log" 2>&1
  else
    python "$@" > "$OUT/$log" 2>&1
  fi
  echo "[$log] exit code $?"
}
launch fluidmoe_full.log examples/pretrain_fluidmoe.py $SHAPE --arch matched --mode full --comm auto
launch fluidmoe_baseline.log examples/pretrain_fluidmoe.py $SHAPE --arch matched --mode F --comm a2a
launch megatron.log examples/pretrain_megatron.py $SHAPE
launch deepspeed.log examples/pretrain_deepspeed.py $SHAPE
if [ -d baseline/_ref/fluid ] && [ "$NGPU" -gt 1 ]; then
  launch reference_parity.log -m fluidmoe_b200.tools.parity_reference --layers "$LAYERS" --steps "$STEPS" --lr "$LR"
fi
python - "$OUT" <<'PY'
import glob, os, re, statistics, sys
out = sys.argv[1]
pat = re.compile(r"iteration\s+(\d+)/.*?\(ms\): ([\d.]+).*?lm loss: ([\d.E+-]+)(?:.*?grad norm: ([\d.]+))?")
print(f"{'arm':22s} {'steps':>5s} {'final lm loss':>14s} {'grad norm':>10s} {'median ms/iter':>15s}")
for path in sorted(glob.glob(os.path.join(out, "*.log"))):
    name = os.path.basename(path)[:-4]
    text = open(path, errors="replace").read()
    rows = pat.findall(text)
    if rows:
        ms = statistics.median(float(r[1]) for r in rows[len(rows) // 4:])
        last = rows[-1]
        print(f"{name:22s} {len(rows):5d} {float(last[2]):14.5f} {last[3] or '-':>10s} {ms:15.1f}")
        continue
    m = re.search(r"PARITY_RESULT (\{.*\})", text)
    if m:
        import json
        r = json.loads(m.group(1))
        print(f"{name:22s} {len(r['loss_ours']):5d} ours {r['loss_ours'][-1]:.5f} / reference {r['loss_reference'][-1]:.5f}; "
              f"step-0 output error {r['y_err']:.2e}, worst gradient error {r['worst_grad_err']:.2e}")
        continue
    why = re.search(r"(baseline unavailable: .*)", text)
    print(f"{name:22s}     - {why.group(1) if why else 'no log lines (see ' + path + ')'}")
PY
