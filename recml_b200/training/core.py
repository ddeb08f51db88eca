"""Trainer contract, experiment runner and on-disk layout constants.

Mirrors `recml/core/training/core.py:38-195`: the directory names below are part of
the checkpoint/log layout that other tools read, so their VALUES are kept verbatim.
"""
from __future__ import annotations

import abc
import dataclasses
import enum
from typing import Any, Generic, Mapping, Sequence, TypeVar

from recml_b200.data import iterator as iterator_lib

LOG_DIR = "logs"
BACKUP_DIR = "backup"
CHECKPOINT_DIR = "checkpoints"
TRAINING_COMPLETE_MARKER_FILE = "marker.txt"
TRAIN_LOG_DIRNAME = "train"
EVAL_LOG_DIRNAME = "val"
KERAS_MODEL_SAVEFILE = "model.keras"
MODULE_SAVEFILE = "model.pt"
ORBAX_CHECKPOINT_DEFAULT_KEY = "default"
STATE_CHECKPOINT_KEY = "state"
DEFAULT_RNG_SEED = 0

TaskT = TypeVar("TaskT")
Logs = Any


class Trainer(abc.ABC, Generic[TaskT]):
  """Interface every trainer implements: four run modes over a task."""

  @abc.abstractmethod
  def __init__(self, model_dir: str, *args, **kwargs): ...

  @abc.abstractmethod
  def train(self, task: TaskT, *args, **kwargs) -> Logs | None: ...

  @abc.abstractmethod
  def evaluate(self, task: TaskT, *args, **kwargs) -> Logs | None: ...

  @abc.abstractmethod
  def train_and_evaluate(self, task: TaskT, *args, **kwargs) -> Logs | None: ...

  @abc.abstractmethod
  def evaluate_continuously(self, task: TaskT, *args, **kwargs) -> Logs | None: ...


@dataclasses.dataclass(frozen=True)
class Experiment(Generic[TaskT]):
  """A task (what to compute) paired with a trainer (how to run it)."""

  class Mode(enum.StrEnum):
    TRAIN = "train"
    EVAL = "eval"
    TRAIN_AND_EVAL = "train_and_eval"
    CONTINUOUS_EVAL = "continuous_eval"

  task: TaskT
  trainer: Trainer[TaskT]


def run_experiment(experiment: Experiment, mode: Experiment.Mode | str) -> Logs | None:
  mode = Experiment.Mode(mode)
  fn = {
      Experiment.Mode.TRAIN: experiment.trainer.train,
      Experiment.Mode.EVAL: experiment.trainer.evaluate,
      Experiment.Mode.TRAIN_AND_EVAL: experiment.trainer.train_and_evaluate,
      Experiment.Mode.CONTINUOUS_EVAL: experiment.trainer.evaluate_continuously,
  }[mode]
  return fn(experiment.task)


def _as_iterator(ds: Any) -> iterator_lib.Iterator:
  if isinstance(ds, iterator_lib.Iterator):
    return ds
  if hasattr(ds, "__iter__") or hasattr(ds, "__next__"):
    return iterator_lib.IterableIterator(ds)
  raise ValueError(f"Expected an Iterator or an iterable dataset, got {type(ds)}.")


def get_iterators(datasets: Any) -> tuple[iterator_lib.Iterator, Mapping[str, iterator_lib.Iterator]]:
  """Normalises what `create_datasets` returned into (train_iter, {name: eval_iter}).

  Accepted: a single dataset; `(train, eval)`; `(train, {name: eval})`.  A single
  unnamed eval set is keyed by "" so that its log dir is plain "val".
  """
  if not isinstance(datasets, tuple):
    return _as_iterator(datasets), {}
  if len(datasets) != 2:
    raise ValueError("Expected `datasets` to be a single dataset or a (train, eval) tuple, "
                     f"got a tuple of length {len(datasets)}.")
  train, evals = datasets
  train = _as_iterator(train)
  if isinstance(evals, Mapping):
    return train, {k: _as_iterator(v) for k, v in evals.items()}
  return train, {"": _as_iterator(evals)}


def get_shape(x: Any) -> Sequence[int | None]:
  """Static shape of a dense / jagged tensor or spec; jagged inner dims are None."""
  if hasattr(x, "values") and hasattr(x, "offsets") and callable(getattr(x, "batch_size", None)):
    return [x.batch_size(), None]
  return list(x.shape)


def in_tracing_context() -> bool:
  """True while a CUDA graph is being captured (the analogue of "under jit trace")."""
  import torch
  return torch.cuda.is_available() and torch.cuda.is_current_stream_capturing()
