"""HSTU generative-retrieval experiment (counterpart of `recml/examples/train_hstu_jax.py:98-236`
and `train_hstu_keras.py:149-195`) on synthetic packed sequences: power-law lengths in [16, 4096]
with mean ≈ 512, Zipf item ids over a 10 M vocabulary, Exponential(1 h) timestamp gaps, sampled
softmax with 512 shared uniform negatives + in-batch negatives."""
from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from recml_b200 import config as cfg_lib
from recml_b200 import embedding as emb
from recml_b200 import metrics as M
from recml_b200.data import iterator as iterator_lib
from recml_b200.data import synthetic
from recml_b200.models import hstu_retrieval
from recml_b200.training import core, optim_factory, partitioning, state as state_lib, task as task_lib
from recml_b200.training import trainer as trainer_lib
from recml_b200.utils import types


@dataclasses.dataclass
class HSTUModelConfig:
  vocab_size: int = 10_000_000
  model_dim: int = 256
  num_heads: int = 4
  num_layers: int = 8
  max_seq_len: int = 4096
  min_seq_len: int = 16
  mean_seq_len: int = 512
  sequences_per_batch: int = 128      # per process
  token_capacity: int = 98304         # per process; batches are generated to fit
  num_negatives: int = 512
  num_in_batch: int = 512
  embedding_learning_rate: float = 0.01
  learning_rate: float = 1e-3
  backend: str = "auto"


class PackedSequenceFactory(types.Factory[Any]):
  model: HSTUModelConfig
  num_batches: int = 4
  steps: int | None = None
  seed: int = 0

  def make(self):
    c = self.model
    rank = dist.get_rank() if dist.is_initialized() else 0
    rng = np.random.default_rng(self.seed * 7919 + rank)
    batches = [synthetic.make_hstu_batch(
        rng, c.sequences_per_batch, c.vocab_size, min_len=c.min_seq_len, max_len=c.max_seq_len,
        mean_target=c.mean_seq_len, num_negatives=c.num_negatives, token_capacity=c.token_capacity)
               for _ in range(self.num_batches)]
    # shared negatives must be identical on all ranks: draw them from a rank-independent stream
    shared = np.random.default_rng(self.seed + 12345)
    for b in batches:
      b["negative_ids"] = torch.from_numpy(shared.integers(0, c.vocab_size, c.num_negatives).astype(np.int32))
    steps = self.steps

    class _Cycle:
      def __iter__(self_inner):
        i = 0
        while steps is None or i < steps:
          yield batches[i % len(batches)]
          i += 1
    return iterator_lib.IterableIterator(_Cycle())


class HSTUTask(task_lib.Task):
  def __init__(self, model: HSTUModelConfig, train_data: PackedSequenceFactory,
               eval_data: PackedSequenceFactory | None = None, group=None):
    self.cfg, self.train_data, self.eval_data, self.group = model, train_data, eval_data, group

  def create_datasets(self):
    tr = self.train_data.make()
    return tr if self.eval_data is None else (tr, self.eval_data.make())

  def create_state(self, batch, rng) -> state_lib.State:
    c = self.cfg
    device = batch["input_ids"].device
    torch.manual_seed(rng.initial_seed())
    model = hstu_retrieval.HSTURetrieval(
        vocab_size=c.vocab_size, model_dim=c.model_dim, num_heads=c.num_heads, num_layers=c.num_layers,
        max_seq_len=c.max_seq_len, token_capacity=c.token_capacity, num_negatives=c.num_negatives,
        num_in_batch=c.num_in_batch, device=device, group=self.group, backend=c.backend,
        embedding_optimizer=emb.RowWiseAdagradOptimizerSpec(c.embedding_learning_rate), seed=rng.initial_seed())
    return state_lib.State.create(model=model, tx=optim_factory.AdamFactory(learning_rate=c.learning_rate).make())

  @staticmethod
  def _args(batch):
    return (batch["input_ids"], batch["target_ids"], batch["negative_ids"], batch["seq_offsets"],
            batch["timestamps"], batch["target_weights"])

  def export_model(self, state, model_dir: str) -> None:
    """`<model_dir>/export` for `recml_b200.serving.load` (collective: every rank writes its table shards)."""
    import os
    from recml_b200 import serving
    c = self.cfg
    serving.export(state.model, os.path.join(model_dir, "export"),
                   builder="recml_b200.models.hstu_retrieval:HSTURetrieval",
                   kwargs=dict(vocab_size=c.vocab_size, model_dim=c.model_dim, num_heads=c.num_heads,
                               num_layers=c.num_layers, max_seq_len=c.max_seq_len, token_capacity=c.token_capacity,
                               num_negatives=c.num_negatives, num_in_batch=c.num_in_batch, backend=c.backend),
                   step=state.step)

  def train_step(self, batch, state, rng):
    state.model.train()
    loss, hit = state.model(*self._args(batch))
    loss.backward()
    state.update()
    n = batch["target_weights"].sum()
    return state, {"loss": M.Mean(total=loss.detach() * n, count=n), "hit@1_sampled": M.Mean(total=hit * n, count=n),
                   "tokens": M.Sum(total=torch.tensor(float(batch["input_ids"].numel())))}

  def eval_step(self, batch, state):
    state.model.eval()
    loss, hit = state.model(*self._args(batch))
    n = batch["target_weights"].sum()
    return {"loss": M.Mean(total=loss.detach() * n, count=n), "hit@1_sampled": M.Mean(total=hit * n, count=n)}


def experiment(model_dir: str = "/tmp/hstu", train_steps: int = 2000) -> cfg_lib.Config:
  model = cfg_lib.Config(HSTUModelConfig)
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(HSTUTask, model=model, train_data=cfg_lib.Config(PackedSequenceFactory, model=model),
                          eval_data=cfg_lib.Config(PackedSequenceFactory, model=model, steps=10, seed=1)),
      trainer=cfg_lib.Config(trainer_lib.Trainer, partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=10, steps_per_eval=10))


def tiny_experiment(model_dir: str = "/tmp/hstu_tiny", train_steps: int = 40) -> cfg_lib.Config:
  model = cfg_lib.Config(HSTUModelConfig, vocab_size=2000, model_dim=64, num_heads=1, num_layers=2, max_seq_len=256,
                         min_seq_len=4, mean_seq_len=40, sequences_per_batch=8, token_capacity=1024,
                         num_negatives=32, num_in_batch=32, learning_rate=3e-3, embedding_learning_rate=0.05)
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(HSTUTask, model=model, train_data=cfg_lib.Config(PackedSequenceFactory, model=model, num_batches=2),
                          eval_data=cfg_lib.Config(PackedSequenceFactory, model=model, steps=2, seed=1, num_batches=2)),
      trainer=cfg_lib.Config(trainer_lib.Trainer, partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=20, steps_per_eval=2))
