"""Command-line launcher for the experiment-based examples.

    python -m torch.distributed.run --nproc-per-node 8 -m recml_b200.examples.run \
        --experiment="config:recml_b200.examples.hstu_experiment.experiment" \
        --experiment="set:trainer.model_dir='/data/hstu'" --experiment="set:trainer.train_steps=5000" \
        --mode=train_and_eval

`--experiment` takes the `config:` / `fiddler:` / `set:` directives of the reference's Fiddle flag
(`recml/core/utils/config.py:28-68`; the example mains `recml/examples/train_hstu_jax.py:238-262`,
`train_hstu_keras.py` and `dlrm_experiment.py` build one experiment and run it).  The process
group is created here from the torchrun environment, one process per GPU.
"""
from __future__ import annotations

import os

from absl import app
from absl import flags
from absl import logging
import torch
import torch.distributed as dist

from recml_b200 import config as config_lib
from recml_b200.training import core

FLAGS = flags.FLAGS
_EXPERIMENT = config_lib.DEFINE_fiddle_config(
    "experiment", help_string="Experiment config: config:<module.fn>, then fiddler:/set: directives.", required=True)
# (allow_override: the standalone DLRM trainer has a --mode of its own; importing both modules must not fail)
flags.DEFINE_enum("mode", "train_and_eval", [m.value for m in core.Experiment.Mode], "What to run.", allow_override=True)


def init_distributed() -> None:
  if "RANK" not in os.environ or dist.is_initialized():
    return
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  if torch.cuda.is_available():
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
  else:
    dist.init_process_group("gloo")


def main(argv):
  del argv
  init_distributed()
  cfg = _EXPERIMENT.value
  experiment = config_lib.build(cfg)
  logs = core.run_experiment(experiment, FLAGS.mode)
  if not dist.is_initialized() or dist.get_rank() == 0:
    for split, values in (logs or {}).items():
      if isinstance(values, dict):
        logging.info("%s: %s", split, {k: (float(v) if hasattr(v, "__float__") else v) for k, v in values.items()})
  if dist.is_initialized():
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
  app.run(main)
