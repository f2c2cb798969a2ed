#!/usr/bin/env bash
# Every arm of the block benchmark on this node: this framework's three scheduler modes, the
# reference implementation (when installed under baseline/_ref), this framework in the
# reference-expressible configuration, then the exposed-communication report; a table of forward
# and iteration times with the speed-ups over the non-overlapped arm and over the reference.
#   NGPUS=8 MODELS=cfg23_mixtral_block,cfg5_fine_grained_block fluidmoe_b200/tools/run_all_block_benchmarks.sh
# Multi-node: set NNODES, NODE_RANK, MASTER_ADDR, MASTER_PORT as for torchrun.
# The exit code is 0 only when every job that could run succeeded (as in the reference's driver,
# tests/run_all_block_benchmarks.sh:206-211).
set -uo pipefail
NGPUS=${NGPUS:-8}
MODELS=${MODELS:-${MODEL:-mixtral_8x7b}}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
WARMUP=${WARMUP:-10}; ITERS=${ITERS:-50}
OUT=${OUT:-block_benchmark_results.txt}
cd "$(dirname "$0")/../.."
FAILED=0
run() {
  MASTER_PORT=$((MASTER_PORT + 1))
  python -m torch.distributed.run --nnodes="$NNODES" --node-rank="$NODE_RANK" --nproc-per-node "$NGPUS" \
    --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" -m "$@"
}
job() {  # job <label> <module args...>: append RESULT lines, count failures
  local label=$1; shift
  echo "== $label ==" >&2
  if ! run "$@" 2>&1 | tee /dev/stderr | grep '^RESULT' >> "$OUT"; then
    echo "job '$label' produced no result" >&2
    FAILED=$((FAILED + 1))
  fi
}
: > "$OUT"
COMMON="--model $MODELS --warmup $WARMUP --iters $ITERS"
for impl in fluidmoe-f fluidmoe-fb fluidmoe-full; do
  job "$impl" fluidmoe_b200.tools.run_block_benchmark $COMMON --impl "$impl"
done
if [ -d baseline/_ref/fluid ]; then
  job "reference" fluidmoe_b200.tools.run_block_benchmark $COMMON --impl reference
  job "fluidmoe-full, reference-expressible configuration" fluidmoe_b200.tools.run_block_benchmark $COMMON --impl fluidmoe-full --matched
else
  echo "reference not installed under baseline/_ref: its arm is skipped" >&2
fi
python - "$OUT" <<'PY'
import re, sys
rows = {}
for line in open(sys.argv[1]):
    kv = dict(re.findall(r"(\w+)=([\w.\-]+)", line))
    if "iter_ms" in kv:
        rows.setdefault(kv["model"], {})[kv["impl"]] = kv
for model, res in rows.items():
    print(f"\n{model} ({next(iter(res.values()))['gpus']} GPUs)")
    base, ref = res.get("fluidmoe-f"), res.get("reference")
    for impl, kv in res.items():
        it, fw = float(kv["iter_ms"]), float(kv["forward_ms"])
        extra = ""
        if base:
            extra += f"  x{float(base['iter_ms']) / it:.3f} over fluidmoe-f"
        if ref and impl != "reference":
            extra += f"  x{float(ref['iter_ms']) / it:.3f} over reference (forward x{float(ref['forward_ms']) / fw:.3f})"
        if "exposed_comm_frac" in kv:
            extra += f"  exposed communication {100 * float(kv['exposed_comm_frac']):.1f} %"
        print(f"  {impl:22s} forward {fw:9.3f} ms  iteration {it:9.3f} ms  {float(kv['tokens_per_sec']):12.1f} tokens/s{extra}")
PY
run fluidmoe_b200.tools.overlap_ratio_analyzer --model "${MODELS%%,*}" --comm auto || FAILED=$((FAILED + 1))
exit $((FAILED > 0))
