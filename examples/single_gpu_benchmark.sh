#!/bin/bash
# One-GPU benchmark through the entry point: a few training steps and the device-side throughput the run reports
# (the reference's scripts/single_gpu_benchmark.sh divides tokens by the wall time of the whole process, start-up
# included; here the number comes from the per-step records, the first step left out).
#   NUM_TOKENS=131072 NUM_LAYERS=4 STEPS=5 bash examples/single_gpu_benchmark.sh
# The full headline measurement (Llama-3-8B, 32 layers, 131072 tokens, one JSON line) is `python bench.py --gpus 1`.
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL=${MODEL:-llama3-8b}
NUM_TOKENS=${NUM_TOKENS:-131072}
NUM_LAYERS=${NUM_LAYERS:-4}
STEPS=${STEPS:-5}
OUT=${OUTPUT_DIR:-logs/single_gpu_benchmark}
python -c "import __graft_entry__ as g; g.build()"
python pretrain_llama.py --model "$MODEL" --num-layers "$NUM_LAYERS" --num-tokens "$NUM_TOKENS" --sample-name mixture \
    --max-sample-id "$STEPS" --val-every-n-steps 0 --output-dir "$OUT" ${EXTRA_ARGS:-}
python - "$OUT" <<'PY'
import json, sys
s = json.load(open(sys.argv[1] + "/benchmark.json"))
print(f"=== single-GPU benchmark: {s['steps']} steps, {s['mean_step_ms']:.1f} ms/step, {s['mean_tokens_per_s']:.0f} tokens/s ===")
PY
