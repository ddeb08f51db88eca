"""SASRec experiment: 2 blocks, hidden 256, 4 heads, FFN 1024, learned positions, max length 200,
lengths ~ uniform[5, 200] right-aligned, Zipf(1.1) item ids over a 20 M × 256 row-sharded table; BCE with
one positive and one sampled negative per position; full-vocabulary NDCG@10 / Recall@10 / MRR at eval
(model: `recml/layers/keras/sasrec.py`; the reference has no SASRec example script)."""
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
from recml_b200.metrics import ranking
from recml_b200.models import sasrec_retrieval
from recml_b200.training import core, optim_factory, partitioning, state as state_lib, task as task_lib
from recml_b200.training import trainer as trainer_lib
from recml_b200.utils import types


@dataclasses.dataclass
class SASRecConfig:
  vocab_size: int = 20_000_000
  max_positions: int = 200
  model_dim: int = 256
  mlp_dim: int = 1024
  num_heads: int = 4
  num_layers: int = 2
  batch_size: int = 512            # per process
  min_len: int = 5
  learning_rate: float = 1e-3
  embedding_learning_rate: float = 0.05
  backend: str = "auto"


def make_batch(rng: np.random.Generator, c: SASRecConfig) -> dict:
  B, L = c.batch_size, c.max_positions
  lens = rng.integers(c.min_len, L + 1, B)
  seq = synthetic.zipf_ids(rng, c.vocab_size - 1, (B, L + 1), 1.1) + 1       # id 0 is padding
  mask = (np.arange(L)[None, :] >= (L - lens)[:, None])                      # right-aligned
  return {"input_ids": torch.from_numpy(np.where(mask, seq[:, :L], 0).astype(np.int32)),
          "positive_ids": torch.from_numpy(np.where(mask, seq[:, 1:], 0).astype(np.int32)),
          "negative_ids": torch.from_numpy(np.where(mask, rng.integers(1, c.vocab_size, (B, L)), 0).astype(np.int32)),
          "padding_mask": torch.from_numpy(mask.astype(np.int32))}


class SequenceFactory(types.Factory[Any]):
  model: SASRecConfig
  num_batches: int = 4
  steps: int | None = None
  seed: int = 0

  def make(self):
    rank = dist.get_rank() if dist.is_initialized() else 0
    rng = np.random.default_rng(self.seed * 104729 + rank)
    batches = [make_batch(rng, self.model) for _ in range(self.num_batches)]
    steps = self.steps

    class _Cycle:
      def __iter__(self_inner):
        i = 0
        while steps is None or i < steps:
          yield batches[i % len(batches)]
          i += 1
    return iterator_lib.IterableIterator(_Cycle())


class SASRecTask(task_lib.Task):
  def __init__(self, model: SASRecConfig, train_data: SequenceFactory, eval_data: SequenceFactory | None = None,
               group=None):
    self.cfg, self.train_data, self.eval_data, self.group = model, train_data, eval_data, group

  def create_datasets(self):
    tr = self.train_data.make()
    return tr if self.eval_data is None else (tr, self.eval_data.make())

  def create_state(self, batch, rng):
    c = self.cfg
    torch.manual_seed(rng.initial_seed())
    model = sasrec_retrieval.SASRecRetrieval(
        vocab_size=c.vocab_size, max_positions=c.max_positions, model_dim=c.model_dim, mlp_dim=c.mlp_dim,
        num_heads=c.num_heads, num_layers=c.num_layers, batch_size=c.batch_size, device=batch["input_ids"].device,
        group=self.group, backend=c.backend, seed=rng.initial_seed(),
        embedding_optimizer=emb.RowWiseAdagradOptimizerSpec(c.embedding_learning_rate))
    return state_lib.State.create(model=model, tx=optim_factory.AdamFactory(learning_rate=c.learning_rate).make())

  def train_step(self, batch, state, rng):
    state.model.train()
    loss = state.model(batch["input_ids"], batch["positive_ids"], batch["negative_ids"], batch["padding_mask"])
    loss.backward()
    state.update()
    n = batch["padding_mask"].sum().float()
    return state, {"loss": M.Mean(total=loss.detach() * n, count=n)}

  def export_model(self, state, model_dir: str) -> None:
    """`<model_dir>/export` for `recml_b200.serving.load` (collective: every rank writes its table shards)."""
    import os
    from recml_b200 import serving
    c = self.cfg
    serving.export(state.model, os.path.join(model_dir, "export"),
                   builder="recml_b200.models.sasrec_retrieval:SASRecRetrieval",
                   kwargs=dict(vocab_size=c.vocab_size, max_positions=c.max_positions, model_dim=c.model_dim,
                               mlp_dim=c.mlp_dim, num_heads=c.num_heads, num_layers=c.num_layers,
                               batch_size=c.batch_size, backend=c.backend), step=state.step)

  def eval_step(self, batch, state):
    """Leave-last-out: the history is everything but the final item, the target is the final item."""
    state.model.eval()
    ids, mask = batch["input_ids"], batch["padding_mask"]
    target = batch["positive_ids"][:, -1].long()
    ranks = state.model.evaluate_ranks(ids, mask, target)
    return {"ndcg@10": ranking.ndcg_at_k_from_rank(ranks, 10), "recall@10": ranking.recall_at_k_from_rank(ranks, 10),
            "mrr": ranking.mrr_from_rank(ranks)}


def experiment(model_dir: str = "/tmp/sasrec", train_steps: int = 1000) -> cfg_lib.Config:
  model = cfg_lib.Config(SASRecConfig)
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(SASRecTask, model=model, train_data=cfg_lib.Config(SequenceFactory, model=model),
                          eval_data=cfg_lib.Config(SequenceFactory, model=model, steps=4, seed=1)),
      trainer=cfg_lib.Config(trainer_lib.Trainer, partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=50, steps_per_eval=4))


def tiny_experiment(model_dir: str = "/tmp/sasrec_tiny", train_steps: int = 30) -> cfg_lib.Config:
  model = cfg_lib.Config(SASRecConfig, vocab_size=3000, max_positions=16, model_dim=64, mlp_dim=128, num_heads=2,
                         num_layers=1, batch_size=32, min_len=3)
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(SASRecTask, model=model, train_data=cfg_lib.Config(SequenceFactory, model=model, num_batches=2),
                          eval_data=cfg_lib.Config(SequenceFactory, model=model, steps=2, seed=1, num_batches=2)),
      trainer=cfg_lib.Config(trainer_lib.Trainer, partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=15, steps_per_eval=2))
