"""Standalone DLRM-DCNv2 trainer: flags in, throughput and eval metrics out.

The counterpart of `recml/inference/models/jax/DLRM_DCNv2/dlrm_main.py` (flags `:66-117`, threaded
producer `:174-291`, train loop with periodic log / eval / checkpoint `:359-498`, eval-only restore
`:501-575`), without the experiment / trainer machinery: one process per GPU, launched with
`python -m torch.distributed.run --nproc-per-node N -m recml_b200.examples.dlrm_main --flags…`.
With no `--file_pattern` it trains on synthetic Criteo-shaped batches.  The model emits logits and
the loss is BCE-with-logits (the reference applies a sigmoid and then BCE-with-logits on top).
"""
from __future__ import annotations

import os
import time

from absl import app
from absl import flags
from absl import logging
import numpy as np
import torch
import torch.distributed as dist

from recml_b200 import ckpt as ckpt_lib
from recml_b200 import metrics as M
from recml_b200.data import criteo
from recml_b200.data import synthetic
from recml_b200.examples import dlrm_experiment as D
from recml_b200.metrics import tools as metrics_tools
from recml_b200.training import optim_factory
from recml_b200.training import partitioning

FLAGS = flags.FLAGS
flags.DEFINE_integer("num_dense_features", 13, "Number of dense features.")
flags.DEFINE_integer("embedding_size", 128, "Embedding size.")
flags.DEFINE_integer("embedding_threshold", 0, "Tables with at most this many rows are replicated on every GPU "
                     "instead of sharded (the reference keeps them on the dense cores at 21000).")
flags.DEFINE_enum("mode", "train", ["train", "eval"], "'train', or 'eval' for evaluation only.", allow_override=True)
flags.DEFINE_integer("batch_size", 8192, "Global batch size.")
flags.DEFINE_string("file_pattern", None, "Training TFRecords (pre-batched Criteo); synthetic data when unset.")
flags.DEFINE_float("learning_rate", 0.0034, "Learning rate (dense Adam and embedding Adagrad).")
flags.DEFINE_integer("num_steps", 28000, "Training steps.")
flags.DEFINE_integer("logging_interval", 6000, "Log training metrics every N steps.")
flags.DEFINE_bool("allow_id_dropping", True, "An embedding occurrence list that overflows drops and counts the ids "
                  "that do not fit instead of ending the run.")
flags.DEFINE_string("eval_file_pattern", None, "Evaluation TFRecords.")
flags.DEFINE_integer("eval_interval", 5000, "Evaluate every N steps.")
flags.DEFINE_integer("eval_steps", 0, "Steps per evaluation, 0 for all.")
flags.DEFINE_string("model_dir", "/tmp/dlrm_b200", "Working directory.")
flags.DEFINE_integer("save_checkpoint_interval", 5000, "Checkpoint every N steps.")
flags.DEFINE_bool("restore_checkpoint", False, "Restore from the latest checkpoint.")
flags.DEFINE_float("vocab_scale", 1.0, "Scales every vocabulary (small runs).")
flags.DEFINE_bool("cuda_graph", True, "Replay the training step as CUDA graphs.")
flags.DEFINE_integer("producer_workers", 16, "Input worker threads.")
flags.DEFINE_integer("producer_depth", 256, "Input queue depth.")


class _Running:
  """Running merge of metric states on the device; `compute` is the only host synchronisation."""

  def __init__(self):
    self._m = None

  def add(self, ms) -> None:
    self._m = dict(ms) if self._m is None else metrics_tools.merge_metrics(self._m, ms)

  def compute(self) -> dict[str, float]:
    if self._m is None:
      return {}
    m = {k: v.reduce_across_ranks().localize() for k, v in self._m.items()}
    return {k: float(np.asarray(v)) for k, v in metrics_tools.compute_metrics(m).items()}


def _world():
  if "RANK" in os.environ and not dist.is_initialized():
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if torch.cuda.is_available():
      torch.cuda.set_device(local)
      dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    else:
      dist.init_process_group("gloo")
  if dist.is_initialized():
    return dist.get_rank(), dist.get_world_size()
  return 0, 1


def _loader(pattern, per_rank_batch, cfg, rank, world, training, steps=None):
  if pattern:
    src = criteo.CriteoDataLoader(pattern, per_rank_batch, vocab_sizes=cfg.vocab_sizes, multi_hot_sizes=cfg.bag_sizes,
                                  is_training=training, process_index=rank, process_count=world,
                                  eval_steps=steps if (not training and steps) else None)
  else:
    src = criteo.synthetic_loader(per_rank_batch, cfg.vocab_sizes, cfg.bag_sizes, steps=steps, rank=rank,
                                  seed=0 if training else 1)
  # queued batches sit in pinned memory: keep the queue under 4 GiB whatever the batch size
  batch_bytes = per_rank_batch * (4 * sum(cfg.bag_sizes) + 4 * 13 + 8)
  depth = max(4, min(FLAGS.producer_depth, (4 << 30) // max(1, batch_bytes)))
  return criteo.ThreadedProducer(src, num_workers=FLAGS.producer_workers, depth=depth, pin=torch.cuda.is_available())


def evaluate(task, part, state, loader, max_steps: int) -> dict[str, float]:
  acc = _Running()
  n = 0
  with torch.no_grad():
    for batch in loader:
      acc.add(task.eval_step(part.shard_inputs(batch), state))
      n += 1
      if max_steps and n >= max_steps:
        break
  out = acc.compute()
  logging.info("Evaluation over %d steps: loss=%.5f accuracy=%.5f auc=%.5f", n, out.get("loss", float("nan")),
               out.get("accuracy", float("nan")), out.get("aucroc", 0.5))
  return out


def run() -> dict:
  """Trains or evaluates according to the flags; returns the last result dict."""
  rank, world = _world()
  if FLAGS.batch_size % world:
    raise ValueError(f"batch_size {FLAGS.batch_size} is not divisible by {world} processes")
  per_rank = FLAGS.batch_size // world
  vocab = tuple(max(3, int(v * FLAGS.vocab_scale)) for v in synthetic.CRITEO_VOCAB_SIZES)
  base = D.ModelConfig()
  cfg = D.ModelConfig(vocab_sizes=vocab, embedding_dim=FLAGS.embedding_size, num_dense=FLAGS.num_dense_features,
                      embedding_learning_rate=FLAGS.learning_rate, allow_id_dropping=FLAGS.allow_id_dropping,
                      bottom_mlp_dims=tuple(base.bottom_mlp_dims[:-1]) + (FLAGS.embedding_size,))
  task = D.PredictionTask(cfg, None, None, optim_factory.AdamFactory(learning_rate=FLAGS.learning_rate))
  device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
  part = partitioning.DataParallelPartitioner(device=device, use_cuda_graph=FLAGS.cuda_graph and device.type == "cuda")
  train_loader = _loader(FLAGS.file_pattern, per_rank, cfg, rank, world, True)
  train_it = iter(train_loader)
  first = part.shard_inputs(next(train_it))
  gen = torch.Generator().manual_seed(0)
  state = part.partition_init(lambda b: task.create_state(b, gen))(first)
  mgr = ckpt_lib.CheckpointManager(os.path.join(FLAGS.model_dir, "checkpoints"), max_to_keep=3,
                                   save_interval_steps=1, item_name="state")
  if (FLAGS.restore_checkpoint or FLAGS.mode == "eval") and mgr.latest_step() is not None:
    step = mgr.latest_step()
    logging.info("Found checkpoint at step %d. Restoring...", step)
    state.load_state_dict(mgr.restore(step, target=state.state_dict()))
  if FLAGS.mode == "eval":
    loader = _loader(FLAGS.eval_file_pattern, per_rank, cfg, rank, world, False, FLAGS.eval_steps or 16)
    return evaluate(task, part, state, loader, FLAGS.eval_steps)

  step_rng = torch.Generator(device=device) if device.type == "cuda" else torch.Generator()
  train_step = part.partition_step(lambda b, s: task.train_step(b, s, step_rng), training=True)
  acc = _Running()
  batch = first
  t_last, s_last = time.time(), state.step
  while state.step < FLAGS.num_steps:
    state, ms = train_step(batch, state)
    acc.add(ms)
    step = state.step
    if step < FLAGS.num_steps:
      batch = part.shard_inputs(next(train_it))
    if step % FLAGS.logging_interval == 0 or step == FLAGS.num_steps:
      out = acc.compute()                     # reads the device: the only host sync of the loop
      dt = time.time() - t_last
      n = step - s_last
      logging.info("step %d: loss=%.5f accuracy=%.5f step_time=%.2fms throughput=%.0f samples/s", step,
                   out.get("loss", float("nan")), out.get("accuracy", float("nan")), 1e3 * dt / max(n, 1),
                   FLAGS.batch_size * n / max(dt, 1e-9))
      acc = _Running()
      t_last, s_last = time.time(), step
    if FLAGS.eval_interval and step % FLAGS.eval_interval == 0 and (FLAGS.eval_file_pattern or not FLAGS.file_pattern):
      loader = _loader(FLAGS.eval_file_pattern, per_rank, cfg, rank, world, False, FLAGS.eval_steps or 16)
      evaluate(task, part, state, loader, FLAGS.eval_steps)
      t_last = time.time()
    if FLAGS.save_checkpoint_interval and step % FLAGS.save_checkpoint_interval == 0:
      mgr.save(step, state.state_dict(), force=True)
  mgr.save(state.step, state.state_dict(), force=True)
  mgr.wait_until_finished()
  return {"step": state.step}


def main(argv):
  del argv
  run()


if __name__ == "__main__":
  app.run(main)
