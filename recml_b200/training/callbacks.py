"""Epoch callbacks and selective checkpoint restore for the compile-and-fit trainer.

Counterparts of `recml/core/utils/keras_utils.py`: `EpochOrbaxCheckpointAndRestoreCallback`
(`:140-178`), `restore_keras_model` with its `restore_optimizer_vars / restore_steps /
restore_iterations` switches (`:181-295`) and `EpochSummaryCallback` (`:299-384`).  A callback sees
the `State` being trained instead of a Keras model.
"""
from __future__ import annotations

import os
import time
from typing import Any, Mapping

import torch

from recml_b200 import ckpt as ckpt_lib
from recml_b200.metrics import tools as metrics_tools
from recml_b200.training import core
from recml_b200.training import state as state_lib


class Callback:
  """Hooks called by `ModuleTrainer`; `self.state` is set before `on_train_begin`."""
  state: state_lib.State | None = None

  def set_state(self, state: state_lib.State) -> None:
    self.state = state

  def on_train_begin(self, logs: Mapping[str, Any] | None = None) -> int | None:
    """May return the first epoch to run (a restoring callback does)."""

  def on_epoch_begin(self, epoch: int, logs: Mapping[str, Any] | None = None) -> None: ...

  def on_epoch_end(self, epoch: int, logs: Mapping[str, Any] | None = None) -> None: ...

  def on_train_end(self, logs: Mapping[str, Any] | None = None) -> None: ...

  def on_test_end(self, logs: Mapping[str, Any] | None = None) -> None:
    """After an evaluation pass that is not part of an epoch (`ModuleTrainer.evaluate`)."""


def restore_state(state: state_lib.State, checkpoint_dir: str, step: int | None = None, *,
                  restore_optimizer_vars: bool = True, restore_steps: bool = True,
                  restore_iterations: bool = True,
                  item_name: str = core.ORBAX_CHECKPOINT_DEFAULT_KEY) -> int:
  """Loads a checkpoint into `state`; returns the step that was restored.

  restore_optimizer_vars  False keeps the freshly initialised optimizer slots.
  restore_steps           False restarts the step / epoch counter at 0.
  restore_iterations      False zeroes the optimizer's own step count (the variable that drives
                          learning-rate schedules and Adam bias correction) while keeping the slots;
                          only meaningful with `restore_optimizer_vars=True`.
  Raises FileNotFoundError when the directory holds no checkpoint and ValueError when `step` is
  not among the saved ones.
  """
  steps = ckpt_lib.all_steps(checkpoint_dir) if os.path.isdir(checkpoint_dir) else []
  if not steps:
    raise FileNotFoundError(f"No checkpoints found in {checkpoint_dir}.")
  if step is None:
    step = steps[-1]
  elif step not in steps:
    raise ValueError(f"Step {step} not found in {checkpoint_dir}. Available steps: {steps}")
  mgr = ckpt_lib.CheckpointManager(checkpoint_dir, max_to_keep=None, item_name=item_name)
  restored = mgr.restore(step, target=state.state_dict())
  state.load_state_dict(restored, restore_optimizer=restore_optimizer_vars, restore_step=restore_steps)
  if not restore_steps:
    state.step = 0
  if restore_optimizer_vars and not restore_iterations and state.optimizer is not None:
    state.optimizer.reset_step_count()
  return step


class EpochCheckpointManager(ckpt_lib.CheckpointManager):
  """A checkpoint manager keyed by epoch that saves and restores a training `State` (parameters, buffers,
  optimizer slots; metric accumulators are per epoch and are not saved) — the part of
  `recml/core/utils/keras_utils.py:36-137` that the epoch callback needs."""

  def __init__(self, checkpoint_dir: str, max_to_keep: int = 5, save_interval_epochs: int = 1, **kwargs):
    kwargs.setdefault("item_name", core.ORBAX_CHECKPOINT_DEFAULT_KEY)
    super().__init__(checkpoint_dir, max_to_keep=max_to_keep, save_interval_steps=save_interval_epochs, **kwargs)

  def save_model_variables(self, state: state_lib.State, epoch: int, logs: Mapping[str, Any] | None = None) -> bool:
    return self.save(epoch, state.state_dict(), metrics=dict(logs or {}))

  def restore_model_variables(self, state: state_lib.State, epoch: int) -> state_lib.State:
    return state.load_state_dict(self.restore(epoch, target=state.state_dict()))


class EpochCheckpointAndRestoreCallback(Callback):
  """Restores the newest epoch checkpoint when training begins, saves one per epoch and writes the
  completion marker when training ends."""

  def __init__(self, manager: ckpt_lib.CheckpointManager, marker_path: str | None = None):
    self._mgr = manager
    self._marker = marker_path

  def on_train_begin(self, logs=None) -> int | None:
    latest = self._mgr.latest_step()
    if latest is None:
      return None
    self.state.load_state_dict(self._mgr.restore(latest, target=self.state.state_dict()))
    return latest + 1

  def on_epoch_end(self, epoch, logs=None):
    self._mgr.save(epoch, self.state.state_dict(), metrics=dict(logs or {}))

  def on_train_end(self, logs=None):
    self._mgr.wait_until_finished()
    rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
    if self._marker is not None and rank == 0:
      os.makedirs(os.path.dirname(self._marker) or ".", exist_ok=True)
      with open(self._marker, "w") as f:
        f.write("COMPLETED")


class EpochSummaryCallback(Callback):
  """Epoch-level scalars at step `epoch * steps_per_epoch`: the epoch's metrics under `train`, the `val_*`
  ones under `val`, the parameter counts (trainable, non-trainable, optimizer slots, total) in both, and
  learning rate(s) and steps per second with the training ones (`recml/core/utils/keras_utils.py:299-384`)."""

  def __init__(self, log_dir: str, steps_per_epoch: int, write_steps_per_second: bool = True):
    self._train = metrics_tools.AsyncMultiWriter(log_dir=log_dir, name=core.TRAIN_LOG_DIRNAME)
    self._val = metrics_tools.AsyncMultiWriter(log_dir=log_dir, name=core.EVAL_LOG_DIRNAME)
    self._steps = steps_per_epoch
    self._write_rate = write_steps_per_second
    self._t0 = time.time()
    self._num_params: dict[str, float] | None = None

  def on_epoch_begin(self, epoch, logs=None):
    self._t0 = time.time()

  def _count_params(self) -> dict[str, float]:
    st = self.state
    if st is None:
      return {}
    if self._num_params is None:
      n = {"num_params/trainable": float(st.num_trainable()),
           "num_params/non_trainable": float(st.num_non_trainable()),
           "num_params/optimizer": float(st.optimizer.num_params()) if st.optimizer is not None else 0.0}
      n["num_params/total"] = sum(n.values())
      self._num_params = n
    return self._num_params

  def on_epoch_end(self, epoch, logs=None):
    if not logs:
      return
    step = epoch * self._steps
    train = {k: v for k, v in logs.items() if not k.startswith("val_")}
    val = {k[4:]: v for k, v in logs.items() if k.startswith("val_")}
    st = self.state
    if st is not None and st.optimizer is not None:
      for name, value in st.optimizer.hyperparams.items():
        if "learning_rate" in name:
          train[name] = float(value)
    if self._write_rate:
      train.setdefault("steps_per_second", self._steps / max(time.time() - self._t0, 1e-9))
    if train:
      train.update(self._count_params())
      self._train.write_scalars(step, train)
      self._train.flush()
    if val:
      val.update(self._count_params())
      self._val.write_scalars(step, val)
      self._val.flush()

  def on_test_end(self, logs=None):
    self._val.flush()

  def on_train_end(self, logs=None):
    self._train.flush()
    self._val.flush()


# The reference's names for the same parts (`recml/core/utils/keras_utils.py`).
KerasOrbaxCheckpointManager = EpochCheckpointManager
EpochOrbaxCheckpointAndRestoreCallback = EpochCheckpointAndRestoreCallback
restore_keras_model = restore_state
