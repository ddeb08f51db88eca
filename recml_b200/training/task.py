"""User-facing task contract (`recml/core/training/jax_trainer.py:295-382`)."""
from __future__ import annotations

import abc
from typing import Any, Mapping

import torch

from recml_b200.metrics import base as metrics_base
from recml_b200.training import state as state_lib


class Task(abc.ABC):
  """Defines datasets, state creation and the train / eval step for a trainer."""

  @abc.abstractmethod
  def create_datasets(self) -> Any:
    """A train iterator, `(train, eval)` or `(train, {name: eval})`."""

  @abc.abstractmethod
  def create_state(self, batch: Any, rng: torch.Generator) -> state_lib.State:
    """Builds the initial state from an example (device-resident) batch."""

  @abc.abstractmethod
  def train_step(self, batch: Any, state: state_lib.State, rng: torch.Generator
                 ) -> tuple[state_lib.State, Mapping[str, metrics_base.Metric]]:
    """Forward, backward, `state.update()`; returns the state and metric states."""

  @abc.abstractmethod
  def eval_step(self, batch: Any, state: state_lib.State) -> Mapping[str, metrics_base.Metric]:
    """Forward only; returns metric states."""

  def restore_state(self, state: state_lib.State) -> state_lib.State:
    """Hook to warm-start from user-provided weights before training / evaluation."""
    return state

  def export_model(self, state: state_lib.State, model_dir: str) -> None:
    """Hook called once training completes, on EVERY rank (exporting sharded embedding tables is a
    collective: see `recml_b200.serving.export`); an override that only writes files should do so on
    rank 0."""
    del state, model_dir


JaxTask = Task
