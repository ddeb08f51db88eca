#!/usr/bin/env bash
# DLRM-DCNv2 on the eight GPUs of one box: standalone trainer, Criteo TFRecords (or synthetic data
# when TRAIN_FILES is unset), periodic evaluation and checkpoints.  The counterpart of the
# reference's recml/inference/benchmarks/DLRM_DCNv2/train_and_checkpoint.sh.
set -euo pipefail
GPUS="${GPUS:-8}"
MODEL_DIR="${MODEL_DIR:-/tmp/dlrm_b200}"
ARGS=(--batch_size="${BATCH_SIZE:-65536}" --embedding_size=128 --learning_rate=0.0034
      --num_steps="${NUM_STEPS:-28000}" --logging_interval=500 --eval_interval=1500 --eval_steps=660
      --save_checkpoint_interval=1500 --model_dir="${MODEL_DIR}")
if [[ -n "${TRAIN_FILES:-}" ]]; then ARGS+=(--file_pattern="${TRAIN_FILES}"); fi
if [[ -n "${EVAL_FILES:-}" ]]; then ARGS+=(--eval_file_pattern="${EVAL_FILES}"); fi
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS}" --master-addr 127.0.0.1 \
  --master-port "${PORT:-29500}" -m recml_b200.examples.dlrm_main "${ARGS[@]}" "$@"
