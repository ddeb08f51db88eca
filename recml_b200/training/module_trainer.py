""""Compile-and-fit" trainer over an `nn.Module` (`recml/core/training/keras_trainer.py:43-371`).

A `ModuleTask` supplies a dataset per phase and a model bundled with its loss, optimizer
and metric functions; `ModuleTrainer` runs epochs of `steps_per_loop` steps
(`epochs = train_steps // steps_per_loop`), restores the newest epoch checkpoint when
training begins, saves one checkpoint per epoch under `checkpoints/<epoch>/default`,
writes epoch-level scalars (`num_params/*`, `learning_rate`, `steps_per_second`,
`val_*`) and `marker.txt` at the end, and exports `model.pt` from rank 0.
"""
from __future__ import annotations

import abc
import dataclasses
import gc
import logging as pylogging
import os
import time
from typing import Any, Callable, Mapping, Sequence

import numpy as np
import torch
from torch import nn

from recml_b200 import ckpt as ckpt_lib
from recml_b200.metrics import reduction
from recml_b200.metrics import tools as metrics_tools
from recml_b200.training import callbacks as callbacks_lib
from recml_b200.training import core
from recml_b200.training import optim_factory
from recml_b200.training import partitioning
from recml_b200.training import state as state_lib

log = pylogging.getLogger("recml_b200.module_trainer")


@dataclasses.dataclass
class CompiledModel:
  """A module plus everything `fit` needs (the analogue of `keras.Model.compile`)."""
  module: nn.Module
  loss: Callable[[Any, Any], torch.Tensor]                       # loss(outputs, labels)
  optimizer: optim_factory.OptimizerBuilder | None = None
  metrics: Mapping[str, Callable[[Any, Any], Any]] = dataclasses.field(default_factory=dict)
  split_batch: Callable[[Any], tuple[Any, Any]] = lambda b: (b[0], b[1])


class ModuleTask(abc.ABC):
  @abc.abstractmethod
  def create_dataset(self, training: bool) -> Any: ...

  @abc.abstractmethod
  def create_model(self, **kwargs) -> CompiledModel: ...

  def create_model_for_eval(self) -> CompiledModel:
    return self.create_model()

  def export_model(self, model: CompiledModel, model_dir: str) -> None:
    torch.save(model.module.state_dict(), os.path.join(model_dir, core.MODULE_SAVEFILE))


class ModuleTrainer(core.Trainer[ModuleTask]):
  def __init__(self, *, distribution: partitioning.Partitioner | None = None,
               model_dir: str | None = None, train_steps: int = 0, steps_per_loop: int | None = None,
               steps_per_eval: int | None = None, continuous_eval_timeout: int = 30,
               max_checkpoints_to_keep: int = 5, checkpoint_save_interval_epochs: int = 1,
               rng_seed: int = core.DEFAULT_RNG_SEED, enable_checkpointing: bool = True,
               callbacks: Sequence["callbacks_lib.Callback"] = ()):
    self._partitioner = distribution or partitioning.NullPartitioner()
    self._model_dir = model_dir or "/tmp"
    self._steps_per_epoch = steps_per_loop if steps_per_loop is not None else max(train_steps, 1)
    self._num_epochs = train_steps // self._steps_per_epoch if train_steps else 0
    self._steps_per_eval = steps_per_eval
    self._timeout = continuous_eval_timeout
    self._rng_seed = rng_seed
    self._enable_checkpointing = enable_checkpointing
    self._ckpt_dir = os.path.join(self._model_dir, core.CHECKPOINT_DIR)
    self._max_keep = max_checkpoints_to_keep
    self._interval = checkpoint_save_interval_epochs
    self._callbacks = list(callbacks)

  def _manager(self) -> ckpt_lib.CheckpointManager:
    return ckpt_lib.CheckpointManager(self._ckpt_dir, max_to_keep=self._max_keep,
                                      save_interval_steps=self._interval,
                                      item_name=core.ORBAX_CHECKPOINT_DEFAULT_KEY)

  def _state(self, cm: CompiledModel) -> state_lib.State:
    st = state_lib.State.create(model=cm.module, tx=cm.optimizer)
    wrapped = self._partitioner.partition_init(lambda _: st)
    return wrapped(None)

  def _device(self) -> torch.device:
    return getattr(self._partitioner, "device", torch.device("cpu"))

  # -- fit / evaluate -------------------------------------------------------------------
  def _evaluate(self, cm: CompiledModel, dataset, prefix: str = "") -> dict[str, float]:
    cm.module.eval()
    totals: dict[str, Any] = {}
    n = 0
    it = iter(dataset)
    t0 = time.time()
    with torch.no_grad():
      while self._steps_per_eval is None or n < self._steps_per_eval:
        try:
          batch = next(it)
        except StopIteration:
          break
        x, y = cm.split_batch(self._partitioner.shard_inputs(batch))
        out = cm.module(x)
        ms = {"loss": reduction.mean(cm.loss(out, y))}
        ms.update({k: fn(y, out) for k, fn in cm.metrics.items()})
        totals = metrics_tools.merge_metrics(totals, {k: m.localize() for k, m in ms.items()})
        n += 1
    logs = {prefix + k: float(np.asarray(v)) for k, v in metrics_tools.compute_metrics(totals).items()}
    logs[prefix + "steps_per_second"] = n / max(time.time() - t0, 1e-9)
    return logs

  def _fit(self, task: ModuleTask, with_eval: bool) -> dict[str, list[float]]:
    torch.manual_seed(self._rng_seed)
    cm = task.create_model()
    cm.module.to(self._device())
    state = self._state(cm)
    train_ds = task.create_dataset(training=True)
    eval_ds = task.create_dataset(training=False) if with_eval else None
    mgr = self._manager() if self._enable_checkpointing else None
    first_epoch = 0
    if mgr is not None and mgr.latest_step() is not None:  # restore on train begin
      step = mgr.latest_step()
      state.load_state_dict(mgr.restore(step, target=state.state_dict()))
      first_epoch = step + 1
    train_w = metrics_tools.AsyncMultiWriter(
        log_dir=os.path.join(self._model_dir, core.LOG_DIR), name=core.TRAIN_LOG_DIRNAME)
    val_w = metrics_tools.AsyncMultiWriter(
        log_dir=os.path.join(self._model_dir, core.LOG_DIR), name=core.EVAL_LOG_DIRNAME)
    history: dict[str, list[float]] = {}
    it = iter(train_ds)
    for cb in self._callbacks:
      cb.set_state(state)
      begin = cb.on_train_begin({})
      if begin is not None:
        first_epoch = max(first_epoch, begin)
    for epoch in range(first_epoch, self._num_epochs):
      for cb in self._callbacks:
        cb.on_epoch_begin(epoch, {})
      cm.module.train()
      totals: dict[str, Any] = {}
      t0 = time.time()
      for _ in range(self._steps_per_epoch):
        try:
          batch = next(it)
        except StopIteration:
          it = iter(train_ds)
          batch = next(it)
        x, y = cm.split_batch(self._partitioner.shard_inputs(batch))
        out = cm.module(x)
        loss = cm.loss(out, y)
        loss.backward()
        state.update()
        ms = {"loss": reduction.mean(loss.detach())}
        ms.update({k: fn(y, out.detach()) for k, fn in cm.metrics.items()})
        totals = metrics_tools.merge_metrics(totals, {k: m.localize() for k, m in ms.items()})
      logs = {k: float(np.asarray(v)) for k, v in metrics_tools.compute_metrics(totals).items()}
      logs["steps_per_second"] = self._steps_per_epoch / max(time.time() - t0, 1e-9)
      logs["num_params/trainable"] = float(state.num_trainable())
      logs["num_params/non_trainable"] = float(state.num_non_trainable())
      if state.optimizer is not None:
        logs["learning_rate"] = state.optimizer.hyperparams["learning_rate"]
      train_w.write_scalars(epoch, logs)
      train_w.flush()
      if eval_ds is not None:
        vlogs = self._evaluate(cm, eval_ds, prefix="val_")
        val_w.write_scalars(epoch, {k[4:]: v for k, v in vlogs.items()})
        val_w.flush()
        logs.update(vlogs)
      for k, v in logs.items():
        history.setdefault(k, []).append(v)
      if mgr is not None:
        mgr.save(epoch, state.state_dict())
      for cb in self._callbacks:
        cb.on_epoch_end(epoch, logs)
    if mgr is not None:
      mgr.wait_until_finished()
    for cb in self._callbacks:
      cb.on_train_end({k: v[-1] for k, v in history.items()})
    rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
    if rank == 0:
      os.makedirs(self._model_dir, exist_ok=True)
      with open(os.path.join(self._model_dir, core.TRAINING_COMPLETE_MARKER_FILE), "w") as f:
        f.write("COMPLETED")
      task.export_model(cm, self._model_dir)
    return history

  def train(self, task: ModuleTask) -> core.Logs:
    return self._fit(task, with_eval=False)

  def train_and_evaluate(self, task: ModuleTask) -> core.Logs:
    return self._fit(task, with_eval=True)

  def evaluate(self, task: ModuleTask) -> core.Logs:
    cm = task.create_model_for_eval()
    cm.module.to(self._device())
    if self._enable_checkpointing and ckpt_lib.latest_step(self._ckpt_dir) is not None:
      st = self._state(cm)
      st.load_state_dict(self._manager().restore(None, target=st.state_dict()))
    logs = self._evaluate(cm, task.create_dataset(training=False))
    for cb in self._callbacks:
      cb.on_test_end(logs)
    return logs

  def evaluate_continuously(self, task: ModuleTask) -> core.Logs:
    cm = task.create_model_for_eval()
    cm.module.to(self._device())
    st = self._state(cm)
    dataset = task.create_dataset(training=False)
    marker = os.path.join(self._model_dir, core.TRAINING_COMPLETE_MARKER_FILE)
    val_w = metrics_tools.AsyncMultiWriter(
        log_dir=os.path.join(self._model_dir, core.LOG_DIR), name=core.EVAL_LOG_DIRNAME)
    history: dict[str, list[float]] = {}
    mgr = self._manager()
    for epoch in ckpt_lib.checkpoints_iterator(self._ckpt_dir, timeout=self._timeout,
                                               timeout_fn=lambda: os.path.exists(marker)):
      try:
        st.load_state_dict(mgr.restore(epoch, target=st.state_dict()), restore_optimizer=False)
        logs = self._evaluate(cm, dataset)
        val_w.write_scalars(epoch, logs)
        val_w.flush()
        for k, v in logs.items():
          history.setdefault(k, []).append(v)
      except FileNotFoundError:
        log.info("Checkpoint %s did not finish writing; skipping.", epoch)
      gc.collect()
    return history


KerasTask = ModuleTask
KerasTrainer = ModuleTrainer
