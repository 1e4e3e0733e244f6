#!/bin/bash
#SBATCH --job-name=distca-b200
#SBATCH --nodes=1
#SBATCH --ntasks-per-node=1
#SBATCH --gres=gpu:8
#SBATCH --exclusive
#SBATCH --time=01:00:00
#SBATCH --output=logs/slurm/stdout.%j.log
#SBATCH --error=logs/slurm/stderr.%j.log
#
# Training under Slurm: one torchrun per node (srun --ntasks-per-node=1), rendezvous on the first node.
#   sbatch examples/pretrain_llama.slurm.sh
#   salloc -N 2 --gres=gpu:8 ; NNODES=2 TP_SIZE=2 PP_SIZE=2 bash examples/pretrain_llama.slurm.sh
# Every setting is an environment variable with a default (the interface of the reference's pretrain_llama.sh:
# MODE, TP_SIZE, PP_SIZE, NUM_MICROBATCH, BATCH_SIZE, NUM_TOKENS, MAX_SAMPLE_ID, SAMPLE_NAME, the sampling factors,
# ENABLE_NSYS, EXPERIMENT_LOG_MEMORY_USAGE, EXPERIMENT_NVSHMEM_BUFFER_SIZE_GB).
set -euo pipefail
cd "$(dirname "$0")/.."

NNODES=${NNODES:-${SLURM_NNODES:-1}}
GPUS_PER_NODE=${GPUS_PER_NODE:-8}
MODEL=${MODEL:-llama3-8b}                 # preset name or a directory with a Hugging Face config.json (MODEL_PATH)
MODEL_PATH=${MODEL_PATH:-}
NUM_LAYERS=${NUM_LAYERS:-}
TP_SIZE=${TP_SIZE:-1}
PP_SIZE=${PP_SIZE:-1}
DP_SIZE=$(( NNODES * GPUS_PER_NODE / (TP_SIZE * PP_SIZE) ))
NUM_MICROBATCH=${NUM_MICROBATCH:-$(( PP_SIZE > 1 ? 2 * PP_SIZE : 1 ))}
MODE=${MODE:-distca}                      # distca | baseline (per-document CP) | perseq | wlbllm | local
BATCH_SIZE=${BATCH_SIZE:-1}
NUM_TOKENS=${NUM_TOKENS:-131072}
MAX_SAMPLE_ID=${MAX_SAMPLE_ID:-10}
SAMPLE_NAME=${SAMPLE_NAME:-wlbllm}
UP_SAMPLE_FACTOR=${UP_SAMPLE_FACTOR:-4}
ELONGATE_FACTOR=${ELONGATE_FACTOR:-$(( NUM_TOKENS / 65536 > 1 ? NUM_TOKENS / 65536 : 1 ))}
FILTER_THRESHOLD=${FILTER_THRESHOLD:-65536}
FILTER_RATIO=${FILTER_RATIO:-0.50}
CHANGE_LONG_DOC_RATIO=${CHANGE_LONG_DOC_RATIO:-0.0}
VAL_EVERY_N_STEPS=${VAL_EVERY_N_STEPS:-0}
CKPT_EVERY_N_STEPS=${CKPT_EVERY_N_STEPS:-0}
COMM_BUFFER_GB=${EXPERIMENT_NVSHMEM_BUFFER_SIZE_GB:-4}
OUTPUT_DIR=${OUTPUT_DIR:-logs/$(date +%Y%m%d_%H%M%S).${MODE}.n${NNODES}.tp${TP_SIZE}pp${PP_SIZE}dp${DP_SIZE}.t${NUM_TOKENS}}
MASTER_PORT=${MASTER_PORT:-29500}

case "$MODE" in
  distca)   MODE_ARGS="--cad" ;;
  baseline) MODE_ARGS="--baseline-mode percp" ;;
  perseq)   MODE_ARGS="--baseline-mode perseq" ;;
  wlbllm)   MODE_ARGS="--baseline-mode percp --packing wlb" ;;
  local)    MODE_ARGS="--no-cad" ;;
  *) echo "unknown MODE=$MODE" >&2; exit 2 ;;
esac

ARGS="--num-nodes $NNODES --num-gpus-per-node $GPUS_PER_NODE --tp-size $TP_SIZE --pp-size $PP_SIZE --dp-size $DP_SIZE \
 --num-microbatch $NUM_MICROBATCH --num-batches $BATCH_SIZE --num-tokens $NUM_TOKENS --max-sample-id $MAX_SAMPLE_ID \
 --sample-name $SAMPLE_NAME --up-sample-factor $UP_SAMPLE_FACTOR --elongate-factor $ELONGATE_FACTOR \
 --filter-threshold $FILTER_THRESHOLD --filter-ratio $FILTER_RATIO --change-long-doc-ratio $CHANGE_LONG_DOC_RATIO \
 --val-every-n-steps $VAL_EVERY_N_STEPS --ckpt-every-n-steps $CKPT_EVERY_N_STEPS --comm-buffer-gb $COMM_BUFFER_GB \
 --output-dir $OUTPUT_DIR $MODE_ARGS ${EXTRA_ARGS:-}"
if [ -n "$MODEL_PATH" ]; then ARGS="--model-path $MODEL_PATH $ARGS"; else ARGS="--model $MODEL $ARGS"; fi
if [ -n "$NUM_LAYERS" ]; then ARGS="--num-layers $NUM_LAYERS $ARGS"; fi
if [ "${EXPERIMENT_LOG_MEMORY_USAGE:-0}" = "1" ]; then ARGS="$ARGS --log-memory"; fi
NSYS=""
if [ "${ENABLE_NSYS:-0}" = "1" ]; then ARGS="$ARGS --nvtx"; NSYS="nsys profile -o $OUTPUT_DIR/nsys.%h --trace=cuda,nvtx --force-overwrite=true"; fi

mkdir -p "$OUTPUT_DIR" logs/slurm
if [ -n "${SLURM_JOB_ID:-}" ]; then
  HEAD=$(scontrol show hostnames "$SLURM_JOB_NODELIST" | head -n 1)
  LAUNCH="srun --kill-on-bad-exit=1 --nodes=$NNODES --ntasks-per-node=1"
  RDZV="--nnodes=$NNODES --node-rank=\$SLURM_NODEID --master-addr $HEAD --master-port $MASTER_PORT"
else                                                   # no Slurm: this node only
  LAUNCH="bash -c"
  RDZV="--nnodes=1 --master-addr 127.0.0.1 --master-port $MASTER_PORT"
fi
CMD="$NSYS python -m torch.distributed.run $RDZV --nproc-per-node=$GPUS_PER_NODE --max-restarts=0 pretrain_llama.py $ARGS"
echo "$CMD" | tee "$OUTPUT_DIR/command.txt"
if [ "${DRY_RUN:-0}" = "1" ]; then exit 0; fi
if [ -n "${SLURM_JOB_ID:-}" ]; then $LAUNCH bash -c "$CMD"; else bash -c "$CMD"; fi
# out-of-memory check of the per-rank logs, as the reference's script does after a run
if grep -rl "out of memory" "$OUTPUT_DIR" >/dev/null 2>&1; then echo "a rank ran out of memory: see $OUTPUT_DIR" >&2; exit 3; fi
