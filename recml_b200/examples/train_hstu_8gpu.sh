#!/usr/bin/env bash
# HSTU generative retrieval (sharded 10M x 256 item table, sampled softmax) on one box.
set -euo pipefail
GPUS="${GPUS:-8}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${GPUS}" --master-addr 127.0.0.1 \
  --master-port "${PORT:-29500}" -m recml_b200.examples.run \
  --experiment="config:recml_b200.examples.hstu_experiment.experiment" \
  --experiment="set:trainer.model_dir='${MODEL_DIR:-/tmp/hstu_b200}'" \
  --experiment="set:trainer.train_steps=${NUM_STEPS:-2000}" --mode="${MODE:-train_and_eval}" "$@"
