#!/usr/bin/env bash
# Run every arm of the block benchmark on this node and print the speed-ups over the
# non-overlapped arm, then the overlap analysis.
#   NGPUS=8 MODEL=mixtral_8x7b fluidmoe_b200/tools/run_all_block_benchmarks.sh
# Multi-node: set NNODES, NODE_RANK, MASTER_ADDR, MASTER_PORT as for torchrun.
set -euo pipefail
NGPUS=${NGPUS:-8}
MODEL=${MODEL:-mixtral_8x7b}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
OUT=${OUT:-block_benchmark_results.txt}
run() {
  python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node "$NGPUS" \
    --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" -m "$@"
}
: > "$OUT"
for impl in fluidmoe-f fluidmoe-fb fluidmoe-full; do
  run fluidmoe_b200.tools.run_block_benchmark --model "$MODEL" --impl "$impl" | tee /dev/stderr | grep '^RESULT' >> "$OUT" || true
done
python - "$OUT" <<'PY'
import re, sys
res = {}
for line in open(sys.argv[1]):
    kv = dict(re.findall(r"(\w+)=([\w.\-]+)", line))
    res[kv["impl"]] = kv
base = res.get("fluidmoe-f")
for impl, kv in res.items():
    sp = f"  speed-up over fluidmoe-f: {float(base['iter_ms']) / float(kv['iter_ms']):.3f}x" if base else ""
    print(f"{impl:14s} forward {float(kv['forward_ms']):9.3f} ms  iteration {float(kv['iter_ms']):9.3f} ms  "
          f"{float(kv['tokens_per_sec']):12.1f} tokens/s{sp}")
PY
run fluidmoe_b200.tools.overlap_ratio_analyzer --model "$MODEL" || true
