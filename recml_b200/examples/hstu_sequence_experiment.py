"""Next-item prediction with the dense (padded) HSTU model from TFRecord files, through the compile-and-fit
trainer: the counterpart of the reference's `recml/examples/train_hstu_keras.py:37-195`.

Records are `tf.Example`s with a variable-length int64 `sequence` (the user's item history) and an int64
`target` of length 1.  Sequences are right-padded (and cut to their last `max_sequence_length` items), the
model encodes them with the HSTU stack, the state at the LAST valid position scores the whole vocabulary
and the loss is the sparse categorical cross-entropy against the target.  Unlike the reference, logits
are formed only for that last position (`[B, V]`), never as `[B, L, V]`.

  python -m recml_b200.examples.run \\
      --experiment=config:recml_b200.examples.hstu_sequence_experiment.experiment --mode=train_and_eval
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any

import numpy as np
import torch
from torch import nn

from recml_b200 import config as C
from recml_b200 import metrics as metrics_lib
from recml_b200.data import tfrecord, tfrecord_factory as F
from recml_b200.layers import hstu as hstu_layers
from recml_b200.training import core, module_trainer, optim_factory, partitioning
from recml_b200.training import state as state_lib
from recml_b200.training import task as task_lib
from recml_b200.training import trainer as trainer_lib


@dataclasses.dataclass
class HSTUModelConfig:
  """`train_hstu_keras.py:40-49`."""
  vocab_size: int = 5_000_000
  max_sequence_length: int = 50
  model_dim: int = 64
  num_heads: int = 4
  num_layers: int = 4
  dropout: float = 0.5
  learning_rate: float = 1e-3


def pad_right(values: np.ndarray, lengths: np.ndarray, max_len: int) -> tuple[np.ndarray, np.ndarray]:
  """Jagged rows -> (`[B, max_len]` ids padded with 0 on the right, `[B, max_len]` 0/1 mask); a row longer
  than `max_len` keeps its LAST `max_len` items (the most recent history)."""
  B = len(lengths)
  starts = np.zeros(B + 1, dtype=np.int64)
  np.cumsum(lengths, out=starts[1:])
  keep = np.minimum(lengths, max_len)
  first = starts[1:] - keep                                   # first kept item of every row
  cols = np.arange(max_len)[None, :]
  mask = cols < keep[:, None]
  idx = np.where(mask, first[:, None] + cols, 0)
  ids = np.where(mask, values[idx] if len(values) else 0, 0).astype(np.int64)
  return ids, mask.astype(np.int32)


@dataclasses.dataclass
class SequenceDataFactory:
  """TFRecord files -> ((input_ids, padding_mask), target) batches (`train_hstu_keras.py:52-90`)."""
  input_path: str
  batch_size: int
  max_sequence_length: int
  is_training: bool = True

  def make(self):
    L = self.max_sequence_length

    def to_model_inputs(feats: dict) -> Any:
      ids, mask = pad_right(feats["sequence"]["values"], feats["sequence"]["lengths"], L)
      x = {"input_ids": torch.from_numpy(ids), "padding_mask": torch.from_numpy(mask)}
      return x, torch.from_numpy(np.ascontiguousarray(feats["target"][:, 0]))

    fac = F.TFDatasetFactory(
        input_path=self.input_path, global_batch_size=self.batch_size,
        feature_spec={"sequence": F.VarLenFeature("int64"), "target": F.FixedLenFeature((1,), "int64")},
        shuffle=self.is_training, shuffle_buffer_size=10_000 if self.is_training else 0, repeat=self.is_training,
        postprocessors=[to_model_inputs])
    return fac.make()


class LastPositionHSTU(nn.Module):
  """HSTU encoder whose output is the vocabulary logits at the last valid position of every sequence
  (`train_hstu_keras.py:110-135`)."""

  def __init__(self, cfg: HSTUModelConfig):
    super().__init__()
    self.hstu = hstu_layers.HSTU(vocab_size=cfg.vocab_size, max_positions=cfg.max_sequence_length,
                                 model_dim=cfg.model_dim, num_heads=cfg.num_heads, num_layers=cfg.num_layers,
                                 dropout=cfg.dropout, add_head=False)

  def forward(self, x: dict) -> torch.Tensor:
    ids, mask = x["input_ids"], x["padding_mask"]
    h = self.hstu(ids, padding_mask=mask)                                   # [B, L, D]
    last = (mask.sum(dim=1).clamp(min=1) - 1).long()                        # right padding: last valid = length - 1
    h_last = h[torch.arange(h.shape[0], device=h.device), last]             # [B, D]
    return self.hstu.item_embedding(h_last, reverse=True)                   # [B, V]


class HSTUSequenceTask(module_trainer.ModuleTask):
  def __init__(self, model_config: HSTUModelConfig, train_data: SequenceDataFactory, eval_data: SequenceDataFactory):
    self.config, self.train_data, self.eval_data = model_config, train_data, eval_data

  def create_dataset(self, training: bool):
    return (self.train_data if training else self.eval_data).make()

  def create_model(self, **kwargs) -> module_trainer.CompiledModel:
    ce = nn.CrossEntropyLoss()
    return module_trainer.CompiledModel(
        LastPositionHSTU(self.config), lambda logits, y: ce(logits.float(), y.long()),
        optim_factory.AdamFactory(learning_rate=self.config.learning_rate).make(),
        {"accuracy": lambda y, logits: metrics_lib.accuracy(y.long(), logits.float()),
         "top_10_accuracy": lambda y, logits: metrics_lib.top_k_accuracy(y.long(), logits.float(), k=10)})


class HSTUSequenceStepTask(task_lib.Task):
  """The same model and data under the step-function trainer (`recml/examples/train_hstu_jax.py:60-200`):
  explicit `create_state` / `train_step` / `eval_step` instead of compile-and-fit."""

  def __init__(self, model_config: HSTUModelConfig, train_data: SequenceDataFactory, eval_data: SequenceDataFactory):
    self.config, self.train_data, self.eval_data = model_config, train_data, eval_data

  def create_datasets(self):
    return self.train_data.make(), self.eval_data.make()

  def create_state(self, batch, rng):
    torch.manual_seed(rng.initial_seed())
    model = LastPositionHSTU(self.config).to(batch[1].device)
    return state_lib.State.create(model=model, tx=optim_factory.AdamFactory(learning_rate=self.config.learning_rate).make())

  @staticmethod
  def _metrics(logits, y):
    loss = nn.functional.cross_entropy(logits.float(), y.long())
    n = torch.tensor(float(y.numel()), device=y.device)
    return loss, {"loss": metrics_lib.Mean(total=loss.detach() * n, count=n),
                  "accuracy": metrics_lib.accuracy(y.long(), logits.detach().float())}

  def train_step(self, batch, state, rng):
    state.model.train()
    x, y = batch
    loss, ms = self._metrics(state.model(x), y)
    loss.backward()
    state.update()
    return state, ms

  def eval_step(self, batch, state):
    state.model.eval()
    x, y = batch
    with torch.no_grad():
      return self._metrics(state.model(x), y)[1]


def step_experiment(train_path: str = "/tmp/hstu_train-*.tfrecord", eval_path: str = "/tmp/hstu_eval-*.tfrecord",
                    model_dir: str = "/tmp/hstu_sequence_steps", vocab_size: int = 5_000_000, batch_size: int = 128,
                    train_steps: int = 2000) -> C.Config:
  max_len = 50
  model = C.Config(HSTUModelConfig, vocab_size=vocab_size, max_sequence_length=max_len, model_dim=64, num_layers=4)
  task = C.Config(HSTUSequenceStepTask, model_config=model,
                  train_data=C.Config(SequenceDataFactory, input_path=train_path, batch_size=batch_size,
                                      max_sequence_length=max_len, is_training=True),
                  eval_data=C.Config(SequenceDataFactory, input_path=eval_path, batch_size=batch_size,
                                     max_sequence_length=max_len, is_training=False))
  trainer = C.Config(trainer_lib.Trainer, partitioner=C.Config(partitioning.DataParallelPartitioner), model_dir=model_dir,
                     train_steps=train_steps, steps_per_loop=100, steps_per_eval=10)
  return C.Config(core.Experiment, task=task, trainer=trainer)


def write_synthetic_tfrecords(path: str, num_examples: int, vocab_size: int, max_len: int = 60, seed: int = 0) -> None:
  """Histories whose next item is a fixed function of the last item, so that a model can learn them."""
  rng = np.random.default_rng(seed)
  recs = []
  for _ in range(num_examples):
    n = int(rng.integers(2, max_len))
    seq = rng.integers(1, vocab_size, n)
    recs.append(tfrecord.encode_example({"sequence": [int(v) for v in seq], "target": [int((seq[-1] * 7 + 3) % vocab_size)]}))
  os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
  tfrecord.write_tfrecord(path, recs)


def experiment(train_path: str = "/tmp/hstu_train-*.tfrecord", eval_path: str = "/tmp/hstu_eval-*.tfrecord",
               model_dir: str = "/tmp/hstu_sequence", vocab_size: int = 5_000_000, batch_size: int = 128,
               train_steps: int = 2000) -> C.Config:
  """`train_hstu_keras.py:149-195`: batch 128, sequences of 50, model dim 64, 4 layers, Adam 1e-3."""
  max_len = 50
  model = C.Config(HSTUModelConfig, vocab_size=vocab_size, max_sequence_length=max_len, model_dim=64, num_layers=4)
  task = C.Config(HSTUSequenceTask, model_config=model,
                  train_data=C.Config(SequenceDataFactory, input_path=train_path, batch_size=batch_size,
                                      max_sequence_length=max_len, is_training=True),
                  eval_data=C.Config(SequenceDataFactory, input_path=eval_path, batch_size=batch_size,
                                     max_sequence_length=max_len, is_training=False))
  trainer = C.Config(module_trainer.ModuleTrainer, model_dir=model_dir, train_steps=train_steps, steps_per_loop=100,
                     steps_per_eval=10)
  return C.Config(core.Experiment, task=task, trainer=trainer)
