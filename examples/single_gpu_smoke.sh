#!/bin/bash
# One-GPU smoke run: build, one tiny training step through every kernel, the GPU kernel tests and one step of the
# entry point (1 layer, 1024 tokens), as the reference's scripts/single_gpu_smoke.sh does for its stack.
set -euo pipefail
cd "$(dirname "$0")/.."
python -c "import __graft_entry__ as g; g.build(); g.smoke()"
python -m pytest tests -q -m gpu -x
python pretrain_llama.py --model tiny-128 --num-tokens 1024 --num-layers 1 --max-sample-id 1
echo "smoke passed"
