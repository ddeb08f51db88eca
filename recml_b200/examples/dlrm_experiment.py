"""DLRM-DCNv2 experiment: task, synthetic Criteo-shaped data and `experiment()` configs.

Counterpart of `recml/examples/dlrm_experiment.py:238-405` (prediction task with BCE loss and the
metrics loss / accuracy / auc (PR) / aucroc / label mean / prediction mean / batch size) using this
framework's trainer, partitioners and sharded embeddings.  `tiny_experiment()` is the CPU
configuration (8 tables × 1000 × 16, bottom 13-64-16, two full-rank cross layers on the 144-d
concat, top 64-1, batch 256, Adagrad 0.01); `experiment()` is the full Criteo-1TB geometry.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Mapping, Sequence

import numpy as np
import torch
import torch.distributed as dist

from recml_b200 import config as cfg_lib
from recml_b200 import embedding as emb
from recml_b200 import metrics as M
from recml_b200.data import iterator as iterator_lib
from recml_b200.data import synthetic
from recml_b200.models import dlrm
from recml_b200.ops import bce
from recml_b200.training import core, optim_factory, partitioning, state as state_lib, task as task_lib
from recml_b200.training import trainer as trainer_lib
from recml_b200.utils import types


@dataclasses.dataclass
class Feature:
  name: str


@dataclasses.dataclass
class DenseFeature(Feature):
  """One scalar input of the bottom MLP."""


@dataclasses.dataclass
class SparseFeature(Feature):
  """One categorical input with a table of its own (`recml/examples/dlrm_experiment.py:57-66`); `bag_size` ids
  per sample are pooled with `combiner`."""
  vocab_size: int = 0
  embedding_dim: int = 128
  max_sequence_length: int | None = None
  combiner: str = "mean"
  sparsity: float = 0.8
  bag_size: int = 1


class FeatureSet:
  """An ordered collection of uniquely named features (`recml/examples/dlrm_experiment.py:68-98`)."""

  def __init__(self, features: Sequence[Feature]):
    self.features = list(features)
    names = [f.name for f in self.features]
    if len(names) != len(set(names)):
      raise ValueError(f"Feature names must be unique. Got names: {names}.")

  def dense_features(self) -> "FeatureSet":
    return FeatureSet([f for f in self if isinstance(f, DenseFeature)])

  def sparse_features(self) -> "FeatureSet":
    return FeatureSet([f for f in self if isinstance(f, SparseFeature)])

  def __iter__(self):
    return iter(self.features)

  def __len__(self) -> int:
    return len(self.features)

  def __or__(self, other: "FeatureSet") -> "FeatureSet":
    return FeatureSet([*self.features, *other.features])


def features(embedding_dim: int = 128) -> FeatureSet:
  """The Criteo-1TB feature set: 13 dense features and 26 categorical ones with the benchmark's vocabulary and
  multi-hot sizes."""
  dense = [DenseFeature(f"float-feature-{i}") for i in range(13)]
  sparse = [SparseFeature(f"categorical-feature-{14 + i}", vocab_size=v, embedding_dim=embedding_dim, bag_size=b)
            for i, (v, b) in enumerate(zip(synthetic.CRITEO_VOCAB_SIZES, synthetic.CRITEO_MULTI_HOT_SIZES))]
  return FeatureSet(dense) | FeatureSet(sparse)


@dataclasses.dataclass
class ModelConfig:
  vocab_sizes: Sequence[int] = synthetic.CRITEO_VOCAB_SIZES
  bag_sizes: Sequence[int] = synthetic.CRITEO_MULTI_HOT_SIZES
  embedding_dim: int = 128
  num_dense: int = 13
  placement_statistics: bool = False    # plan the table placement from statistics of the first batch
  bottom_mlp_dims: Sequence[int] = (512, 256, 128)
  top_mlp_dims: Sequence[int] = (1024, 1024, 512, 256, 1)
  num_cross_layers: int = 3
  cross_rank: int | None = 512
  embedding_learning_rate: float = 0.01
  embedding_init_scale: float | None = None
  row_wise_min_bytes: int | None = None
  backend: str = "auto"
  # an occurrence list that overflows drops (and counts) the ids that do not fit instead of raising
  allow_id_dropping: bool = False

  @classmethod
  def from_features(cls, feature_set: FeatureSet, **kwargs) -> "ModelConfig":
    """The geometry a `FeatureSet` describes: one table per sparse feature (all of one embedding width, which
    the interaction layer needs), the dense features as the bottom MLP's input."""
    sparse = list(feature_set.sparse_features())
    dims = {f.embedding_dim for f in sparse}
    if len(dims) != 1:
      raise ValueError(f"all sparse features must share one embedding_dim, got {sorted(dims)}")
    return cls(vocab_sizes=tuple(f.vocab_size for f in sparse), bag_sizes=tuple(f.bag_size for f in sparse),
               embedding_dim=dims.pop(), num_dense=len(feature_set.dense_features()), **kwargs)


class CriteoFactory(types.Factory[Any]):
  """Synthetic Criteo-shaped batches (Zipf ids, log-normal dense, Bernoulli(0.25) labels)."""
  model: ModelConfig
  batch_size: int            # per process
  num_batches: int = 4
  steps: int | None = None
  seed: int = 0
  alpha: float = 1.05

  def make(self):
    rank = dist.get_rank() if dist.is_initialized() else 0
    ds = synthetic.SyntheticDLRMDataset(
        self.batch_size, self.model.vocab_sizes, self.model.bag_sizes, num_batches=self.num_batches,
        seed=self.seed, rank=rank, alpha=self.alpha, steps=self.steps, num_dense=self.model.num_dense,
        pin=torch.cuda.is_available())
    return iterator_lib.IterableIterator(ds)


@dataclasses.dataclass
class CriteoExampleFactory(types.Factory[Any]):
  """Per-example Criteo `tf.Example` files (`label`, `dense` = 13 floats, `cat_0` .. `cat_25` = id lists) read
  through the native TFRecord factory.  The host id pipeline finishes every batch: it packs the categorical
  features into the jagged layout the sharded embedding consumes, in the embedding's feature order, and (with
  `stats_dir`) keeps the per-table maxima of ids and unique ids per shard that feedback-directed sizing reads
  back (`StatsRecorder.load`)."""
  model: ModelConfig
  input_path: str
  batch_size: int            # global
  is_training: bool = True
  stats_dir: str | None = None

  def make(self):
    from recml_b200.data import tfrecord_factory as F
    from recml_b200.embedding import id_pipeline
    n_cat = len(self.model.vocab_sizes)
    names = [f"cat_{i}" for i in range(n_cat)]
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    recorder = id_pipeline.StatsRecorder(self.stats_dir, rank) if self.stats_dir else None
    pack = id_pipeline.ShardedPreprocessor(names, output_key="sparse", world=world, recorder=recorder,
                                           pin=torch.cuda.is_available())

    def finish(feats: dict) -> dict:
      out = pack(feats)
      out["dense"] = torch.from_numpy(np.ascontiguousarray(out["dense"], dtype=np.float32))
      out["label"] = torch.from_numpy(np.ascontiguousarray(out["label"], dtype=np.float32).reshape(-1))
      return out

    spec = {"label": F.FixedLenFeature((1,), "float32"), "dense": F.FixedLenFeature((self.model.num_dense,), "float32")}
    spec.update({n: F.VarLenFeature("int64") for n in names})
    fac = F.TFDatasetFactory(input_path=self.input_path, global_batch_size=self.batch_size, feature_spec=spec,
                             shuffle=self.is_training, shuffle_buffer_size=10_000 if self.is_training else 0,
                             repeat=self.is_training, postprocessors=[finish])
    it = fac.make()
    it.stats_recorder = recorder
    return it


class PredictionTask(task_lib.Task):
  def __init__(self, model: ModelConfig, train_data: CriteoFactory, eval_data: CriteoFactory | None,
               optimizer: types.Factory, group=None):
    self.cfg, self.train_data, self.eval_data, self.optimizer = model, train_data, eval_data, optimizer
    self.group = group

  def create_datasets(self):
    train = self.train_data.make()
    return train if self.eval_data is None else (train, self.eval_data.make())

  def create_state(self, batch, rng) -> state_lib.State:
    c = self.cfg
    device = batch["dense"].device
    torch.manual_seed(rng.initial_seed())
    # Optional placement statistics from this first batch (a collective: every rank contributes its share and all
    # derive the same plan): ids and distinct ids of every feature per residue class of the row sharding.  Off by
    # default: on the Criteo geometry at 8 GPUs the plan it produces (a third table row-sharded, update kernels
    # within 635 - 800 us instead of 567 - 857 us) lost more in the lookup and the gradient push than it gained
    # (2.93 against 2.88 ms per step).
    stats = None
    if c.placement_statistics or os.environ.get("RECML_PLAN_STATS", "0") == "1":
      world = dist.get_world_size(self.group) if dist.is_initialized() else 1
      stats = emb.batch_residue_stats(batch["sparse"], world, self.group)
    model = dlrm.DLRMDCNv2(
        vocab_sizes=c.vocab_sizes, embedding_dim=c.embedding_dim, num_dense=c.num_dense,
        bottom_mlp_dims=c.bottom_mlp_dims, top_mlp_dims=c.top_mlp_dims,
        num_cross_layers=c.num_cross_layers, cross_rank=c.cross_rank, bag_sizes=c.bag_sizes,
        embedding_optimizer=emb.RowWiseAdagradOptimizerSpec(learning_rate=c.embedding_learning_rate),
        device=device, group=self.group, row_wise_min_bytes=c.row_wise_min_bytes, backend=c.backend,
        init_scale=c.embedding_init_scale, seed=rng.initial_seed(), residue_stats=stats,
        allow_id_dropping=c.allow_id_dropping)
    return state_lib.State.create(model=model, tx=self.optimizer.make())

  def _metrics(self, r: bce.BCEResult, n: int) -> Mapping[str, M.Metric]:
    out = {
        "loss": M.Mean(total=r.loss_sum, count=r.weight_sum),
        "accuracy": M.Mean(total=r.correct_sum, count=r.weight_sum),
        "label/mean": M.Mean(total=r.label_sum, count=r.weight_sum),
        "prediction/mean": M.Mean(total=r.pred_sum, count=r.weight_sum),
        "common/batch_size": M.scalar(float(n)),
    }
    if r.hist_pos is not None:
      # both curves keep the loss kernel's histograms as their state; the suffix sums run on the host at report time
      out["auc"] = M.HistogramAUCPR(pos_hist=r.hist_pos, neg_hist=r.hist_neg)
      out["aucroc"] = M.HistogramAUCROC(pos_hist=r.hist_pos, neg_hist=r.hist_neg)
    return out

  def train_step(self, batch, state, rng):
    state.model.train()
    logits = state.model(batch["dense"], batch["sparse"])
    n = logits.numel()
    r = bce.bce_with_logits(logits.detach(), batch["label"], grad_scale=1.0 / n)
    logits.backward(r.dlogits.to(logits.dtype))
    state.update()
    return state, self._metrics(r, n)

  def eval_step(self, batch, state):
    state.model.eval()
    logits = state.model(batch["dense"], batch["sparse"])
    return self._metrics(bce.bce_with_logits(logits, batch["label"]), logits.numel())

  def model_kwargs(self) -> dict[str, Any]:
    """Keyword arguments that rebuild the module (`serving.load` adds device and group)."""
    c = self.cfg
    return dict(vocab_sizes=list(c.vocab_sizes), embedding_dim=c.embedding_dim, num_dense=c.num_dense,
                bottom_mlp_dims=list(c.bottom_mlp_dims), top_mlp_dims=list(c.top_mlp_dims),
                num_cross_layers=c.num_cross_layers, cross_rank=c.cross_rank, bag_sizes=list(c.bag_sizes),
                row_wise_min_bytes=c.row_wise_min_bytes, backend=c.backend, init_scale=c.embedding_init_scale,
                allow_id_dropping=c.allow_id_dropping)

  def export_model(self, state, model_dir: str) -> None:
    """Writes `<model_dir>/export`: the module's weights (tables shard by shard) and the recipe to rebuild
    it for serving (`recml_b200.serving.load`).  Collective: every rank of the job calls it."""
    import os
    from recml_b200 import serving
    serving.export(state.model, os.path.join(model_dir, "export"), builder="recml_b200.models.dlrm:DLRMDCNv2",
                   kwargs=self.model_kwargs(), step=state.step)


def features_summary(c: ModelConfig) -> str:
  return f"{len(c.vocab_sizes)} tables, {sum(c.bag_sizes)} ids/sample, dim {c.embedding_dim}"


def experiment(global_batch: int = 65536, train_steps: int = 1000, model_dir: str = "/tmp/dlrm") -> cfg_lib.Config:
  """Full Criteo-1TB geometry (bottom 512-256-128, 3 low-rank-512 cross layers, top
  1024-1024-512-256-1; the reference's `experiment()` uses batch 131 072 and Adagrad 0.01)."""
  world = dist.get_world_size() if dist.is_initialized() else 1
  model = cfg_lib.Config(ModelConfig)
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(
          PredictionTask, model=model,
          train_data=cfg_lib.Config(CriteoFactory, model=model, batch_size=global_batch // world),
          eval_data=cfg_lib.Config(CriteoFactory, model=model, batch_size=global_batch // world, steps=8, seed=1),
          optimizer=cfg_lib.Config(optim_factory.AdamFactory, learning_rate=1e-3)),
      trainer=cfg_lib.Config(trainer_lib.Trainer, partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=100, steps_per_eval=8))


def tiny_experiment(model_dir: str = "/tmp/dlrm_tiny", train_steps: int = 100, batch_size: int = 256,
                    ) -> cfg_lib.Config:
  model = cfg_lib.Config(
      ModelConfig, vocab_sizes=(1000,) * 8, bag_sizes=(1,) * 8, embedding_dim=16, bottom_mlp_dims=(64, 16),
      top_mlp_dims=(64, 1), num_cross_layers=2, cross_rank=None, embedding_learning_rate=0.01,
      embedding_init_scale=0.01)
  world = dist.get_world_size() if dist.is_initialized() else 1
  return cfg_lib.Config(
      core.Experiment,
      task=cfg_lib.Config(
          PredictionTask, model=model,
          train_data=cfg_lib.Config(CriteoFactory, model=model, batch_size=batch_size // world, num_batches=8),
          eval_data=cfg_lib.Config(CriteoFactory, model=model, batch_size=batch_size // world, steps=4, seed=1),
          optimizer=cfg_lib.Config(optim_factory.AdagradFactory, learning_rate=0.01)),
      trainer=cfg_lib.Config(trainer_lib.Trainer,
                             partitioner=cfg_lib.Config(partitioning.DataParallelPartitioner),
                             model_dir=model_dir, train_steps=train_steps, steps_per_loop=50, steps_per_eval=4))
