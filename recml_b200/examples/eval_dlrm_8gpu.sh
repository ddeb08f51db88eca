#!/usr/bin/env bash
# Restores the newest checkpoint under MODEL_DIR and evaluates it (the reference's
# recml/inference/benchmarks/DLRM_DCNv2/eval_from_checkpoint.sh).
set -euo pipefail
GPUS="${GPUS:-8}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS}" --master-addr 127.0.0.1 \
  --master-port "${PORT:-29500}" -m recml_b200.examples.dlrm_main --mode=eval \
  --batch_size="${BATCH_SIZE:-65536}" --embedding_size=128 --eval_steps="${EVAL_STEPS:-660}" \
  --model_dir="${MODEL_DIR:-/tmp/dlrm_b200}" ${EVAL_FILES:+--eval_file_pattern="${EVAL_FILES}"} "$@"
