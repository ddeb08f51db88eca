"""Config-driven training / evaluation loops over a `Task`.

Functional parity with the reference's `JaxTrainer`
(`recml/core/training/jax_trainer.py:389-958`): the same constructor arguments, the four
modes, the log-dict keys ("train", "val", "val_<name>"), checkpoint steps
{k·interval−1} ∪ {train_steps−1}, TensorBoard scalars under `<model_dir>/logs/...`,
`marker.txt` on completion and automatic `model/*`, `optimizer/*` and `perf/*` scalars.

Differences that are deliberate:
  * `check_for_checkpoints=True` by default, so `train` resumes from the newest
    checkpoint (the reference passes False everywhere and never auto-resumes).
  * Throughput is also reported from CUDA events (`perf/device_ms_per_step`), because
    wall-clock around an asynchronous GPU stream only measures launch time.
"""
from __future__ import annotations

import functools
import logging as pylogging
import os
import time
from typing import Any, Callable, Mapping

import numpy as np
import torch
import torch.distributed as dist

from recml_b200 import ckpt as ckpt_lib
from recml_b200.metrics import base as metrics_base
from recml_b200.metrics import tools as metrics_tools
from recml_b200.training import core
from recml_b200.training import partitioning
from recml_b200.training import state as state_lib
from recml_b200.training import task as task_lib
from recml_b200.utils import profiling

log = pylogging.getLogger("recml_b200.trainer")
WARMUP_STEPS = 3  # steps excluded from loop throughput (`jax_trainer.py:564-605`)


def _val_logdir(key: str) -> str:
  return f"{core.EVAL_LOG_DIRNAME}_{key}" if key else core.EVAL_LOG_DIRNAME


def _fmt(metrics: Mapping[str, Any]) -> str:
  parts = []
  for k, v in metrics.items():
    a = np.asarray(v)
    parts.append(f"{k}: {float(a):.4f}" if a.size == 1 else f"{k}: {a}")
  return " | ".join(parts)


def _process_index() -> int:
  return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _batch_size_of(batch: Any) -> int:
  if isinstance(batch, dict):
    for v in batch.values():
      n = _batch_size_of(v)
      if n:
        return n
    return 0
  if isinstance(batch, (list, tuple)):
    for v in batch:
      n = _batch_size_of(v)
      if n:
        return n
    return 0
  if hasattr(batch, "batch_size") and callable(batch.batch_size):
    return int(batch.batch_size())
  if hasattr(batch, "shape") and len(batch.shape) >= 1:
    return int(batch.shape[0])
  return 0


def state_metrics(state: state_lib.State) -> dict[str, metrics_base.Metric]:
  """`model/*` and `optimizer/*` scalars logged with every step
  (`jax_trainer.py:903-958`)."""
  out = {
      "model/num_trainable_variables": metrics_base.scalar(float(state.num_trainable())),
      "model/num_non_trainable_variables": metrics_base.scalar(float(state.num_non_trainable())),
  }
  if state.optimizer is not None:
    for k, v in state.optimizer.hyperparams.items():
      out[f"optimizer/{k}"] = metrics_base.scalar(float(v))
    out["optimizer/num_params"] = metrics_base.scalar(float(state.optimizer.num_params()))
  return out


class Trainer(core.Trainer[task_lib.Task]):
  def __init__(self, *, partitioner: partitioning.Partitioner | None = None,
               model_dir: str | None = None, train_steps: int = 0, steps_per_loop: int = 1_000,
               steps_per_eval: int | None = None, checkpoint_interval: int | None = None,
               max_checkpoints_to_keep: int = 5, continuous_eval_timeout: int = 30,
               rng_seed: int = core.DEFAULT_RNG_SEED, rng_impl: str | None = None,
               enable_checkpointing: bool = True, check_for_checkpoints: bool = True,
               failure_detection: bool = False, heartbeat_timeout_s: float = 30.0,
               prefetch_to_device: int = 1):
    if not isinstance(steps_per_loop, int) or steps_per_loop < 1:
      raise ValueError(f"`steps_per_loop` ({steps_per_loop}) must be a positive integer.")
    self._partitioner = partitioner or partitioning.NullPartitioner()
    self._prefetch_depth = prefetch_to_device      # batches copied to the device ahead of the step that uses them
    self._model_dir = model_dir or "/tmp"
    self._train_steps = train_steps
    self._steps_per_loop = steps_per_loop
    self._steps_per_eval = steps_per_eval
    self._continuous_eval_timeout = continuous_eval_timeout
    self._checkpoint_interval = checkpoint_interval or steps_per_loop
    self._max_checkpoints_to_keep = max_checkpoints_to_keep
    self._rng_seed = rng_seed
    self._rng_impl = rng_impl
    self._enable_checkpointing = enable_checkpointing
    self._check_for_checkpoints = check_for_checkpoints
    self._progress = None
    self._failure_detection = failure_detection
    self._heartbeat_timeout_s = heartbeat_timeout_s
    self._health = None

  # -- lazily created helpers ---------------------------------------------------------
  @functools.cached_property
  def checkpoint_manager(self) -> ckpt_lib.CheckpointManager | None:
    if not self._enable_checkpointing:
      return None
    steps = {s for s in range(self._train_steps) if (s + 1) % self._checkpoint_interval == 0}
    steps.add(self._train_steps - 1)  # the final step is always saved
    return ckpt_lib.CheckpointManager(
        os.path.join(self._model_dir, core.CHECKPOINT_DIR),
        max_to_keep=self._max_checkpoints_to_keep,
        should_save_fn=lambda step, _: step in steps, item_name=core.STATE_CHECKPOINT_KEY)

  @functools.cached_property
  def train_summary_writer(self) -> metrics_tools.AsyncMultiWriter:
    return metrics_tools.AsyncMultiWriter(
        log_dir=os.path.join(self._model_dir, core.LOG_DIR), name=core.TRAIN_LOG_DIRNAME)

  @property
  def report_progress(self) -> profiling.ReportProgress:
    """The periodic progress action (`recml/core/training/jax_trainer.py:496-501`): steps per second and uptime
    to the log and to the training summaries, with the share of wall time spent in checkpointing and eval."""
    if self._progress is None:
      self._progress = profiling.ReportProgress(writer=self.train_summary_writer, every_steps=self._steps_per_loop)
    return self._progress

  def _eval_writers(self, eval_iters) -> dict[str, metrics_tools.AsyncMultiWriter]:
    return {k: metrics_tools.AsyncMultiWriter(
        log_dir=os.path.join(self._model_dir, core.LOG_DIR), name=_val_logdir(k))
            for k in eval_iters}

  # -- checkpoints ------------------------------------------------------------------------
  def _maybe_save_checkpoint(self, step: int, state: state_lib.State, metrics=None) -> None:
    mgr = self.checkpoint_manager
    if mgr is None or not mgr.should_save(step):
      return
    if torch.cuda.is_available():
      from recml_b200.ops import _lib
      _lib.check_status()      # raises before anything is written if a kernel reported an error
    with self.report_progress.timed("checkpointing"):
      mgr.save(step, state.state_dict(), metrics=metrics)

  def _maybe_restore_checkpoint(self, state: state_lib.State, step: int | None = None
                                ) -> state_lib.State:
    mgr = self.checkpoint_manager
    if mgr is None:
      return state
    if step is None:
      step = mgr.latest_step()
    if step is None:
      return state
    restored = mgr.restore(step, target=state.state_dict())
    state.load_state_dict(restored)
    log.info("restored checkpoint at step %d", step)
    return state

  def _write_marker_file(self) -> None:
    os.makedirs(self._model_dir, exist_ok=True)
    with open(os.path.join(self._model_dir, core.TRAINING_COMPLETE_MARKER_FILE), "w") as f:
      f.write("COMPLETED")

  # -- failure detection: host heartbeats and a non-blocking look at the device status word between steps;
  #    a blocking check at the end of a loop and before every checkpoint, so that a step whose kernels
  #    reported a timeout, a capacity overflow or a bad index is never saved ---------------------------
  def _start_health(self):
    if not self._failure_detection or self._health is not None:
      return
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
      return
    from recml_b200.comm import health
    store = dist.distributed_c10d._get_default_store()   # pylint: disable=protected-access
    self._health = health.HealthMonitor(store, dist.get_rank(), dist.get_world_size(),
                                        timeout_s=self._heartbeat_timeout_s).start()

  def _check_health(self, step: int, end_of_loop: bool = False) -> None:
    if self._health is not None:
      self._health.check(step)
    if torch.cuda.is_available():
      from recml_b200.ops import _lib
      if end_of_loop:
        _lib.check_status()
      else:
        _lib.poll_status()

  # -- the hot loop ----------------------------------------------------------------------
  def _train_n_steps(self, *, train_iter, train_step, state, start_step: int, num_steps: int,
                     summary_writer) -> tuple[state_lib.State, Mapping[str, Any]]:
    accum = metrics_tools.MetricAccumulator(summary_writer)
    timer = profiling.DeviceStepTimer(enabled=torch.cuda.is_available())
    t0, examples, timed_steps = None, 0, 0
    self._start_health()
    if getattr(self, "_prefetcher_src", None) is not train_iter:       # one prefetcher per iterator, kept across loops
      from recml_b200.data import prefetch
      self._prefetcher = prefetch.DevicePrefetcher(train_iter, self._partitioner, depth=self._prefetch_depth)
      self._prefetcher_src = train_iter
    for step in range(start_step, start_step + num_steps):
      self._check_health(step)
      if step - start_step == WARMUP_STEPS:
        timer.start()
        t0 = time.time()
      with profiling.step_annotation("train", step):
        try:
          inputs, host_batch = self._prefetcher.next_with_host()
        except StopIteration:
          # a bare StopIteration would end any generator above us silently; say what ran out
          raise RuntimeError(f"the training dataset ended at step {step} of {self._train_steps}: repeat it or "
                             "lower `train_steps`") from None
        state, metrics = train_step(inputs, state)
      if t0 is not None:
        examples += _batch_size_of(host_batch)
        timed_steps += 1
      accum.accumulate({**metrics, **state_metrics(state)}, step)
      self.report_progress(step)
      if step != start_step + num_steps - 1:
        self._maybe_save_checkpoint(step, state)
    device_ms = timer.stop()
    self._check_health(start_step + num_steps - 1, end_of_loop=True)
    scalars = dict(accum.compute_and_log_scalars(start_step + num_steps - 1))
    if t0 is not None and timed_steps:
      if torch.cuda.is_available():
        torch.cuda.synchronize()
      dt = max(time.time() - t0, 1e-9)
      perf = {"perf/loop_throughput_ex_per_sec": examples / dt,
              "perf/loop_ms_per_step": 1e3 * dt / timed_steps}
      if device_ms is not None:
        perf["perf/device_ms_per_step"] = device_ms / timed_steps
        perf["perf/device_throughput_ex_per_sec"] = examples / (device_ms * 1e-3)
      summary_writer.write_scalars(start_step + num_steps - 1, perf)
      summary_writer.flush()
      scalars.update(perf)
    return state, scalars

  def _evaluate_n_steps(self, *, eval_iter, eval_step, state, num_steps: int | None,
                        step_number: int, summary_writer) -> Mapping[str, Any]:
    accum = metrics_tools.MetricAccumulator(summary_writer)
    n = 0
    while num_steps is None or n < num_steps:
      try:
        host_batch = next(eval_iter)
      except StopIteration:
        break
      with profiling.step_annotation("eval", n):
        with torch.no_grad():
          metrics = eval_step(self._partitioner.shard_inputs(host_batch), state)
      accum.accumulate(metrics, step_number)
      n += 1
    return accum.compute_and_log_scalars(step_number)

  # -- task set-up -------------------------------------------------------------------------
  def process_task(self, task: task_lib.Task, *, training: bool,
                   check_for_checkpoints: bool | None = None):
    """Builds iterators, initial (possibly restored) state and the partitioned steps."""
    if check_for_checkpoints is None:
      check_for_checkpoints = self._check_for_checkpoints
    device = getattr(self._partitioner, "device", torch.device("cpu"))
    init_rng = torch.Generator(device="cpu").manual_seed(self._rng_seed)
    step_rng = torch.Generator(device=device).manual_seed(self._rng_seed + 1)
    torch.manual_seed(self._rng_seed)
    train_iter, eval_iters = core.get_iterators(task.create_datasets())
    spec_iter = train_iter if training or not eval_iters else next(iter(eval_iters.values()))
    spec_iter.element_spec  # peeks (and caches) the first batch, as the reference does
    example = spec_iter._peeked[0] if getattr(spec_iter, "_peeked", None) else next(spec_iter)
    batch = self._partitioner.shard_inputs(example)

    init_fn = self._partitioner.partition_init(
        lambda b: task.create_state(b, init_rng), abstract_batch=batch)
    state = init_fn(batch)
    state = task.restore_state(state)
    if check_for_checkpoints and self._enable_checkpointing:
      state = self._maybe_restore_checkpoint(state)

    def _train(inputs, st):
      from recml_b200.utils import graphs
      if not graphs.capturing():   # reseeding a CUDA generator is not allowed while a graph records
        step_rng.manual_seed(self._rng_seed + 1 + st.step)  # fold the step into the stream
      return task.train_step(inputs, st, step_rng)

    train_step = self._partitioner.partition_step(_train, training=True)
    eval_step = self._partitioner.partition_step(task.eval_step, training=False)
    return train_iter, eval_iters, state, train_step, eval_step, state.step

  # -- modes ----------------------------------------------------------------------------------
  def _finish_training(self, task, state):
    mgr = self.checkpoint_manager
    if mgr is not None:
      mgr.wait_until_finished()
    if _process_index() == 0:
      self._write_marker_file()
    # The reference calls the hook on process 0 only; here every rank calls it, because an export of
    # sharded tables is collective (each rank writes its shards).  Hooks that only write files guard on rank.
    task.export_model(state, self._model_dir)
    if mgr is not None:
      mgr.close()
      del self.checkpoint_manager

  def _run_evals(self, eval_iters, eval_step, state, step, writers, metrics):
    msg = (f"running {self._steps_per_eval} steps of evaluation..."
           if self._steps_per_eval is not None else "running complete evaluation...")
    log.info("eval | step: %6d | %s", step, msg)
    with self.report_progress.timed("eval"):
      for key, it in eval_iters.items():
        it.reset()
        m = self._evaluate_n_steps(eval_iter=it, eval_step=eval_step, state=state,
                                   num_steps=self._steps_per_eval, step_number=step,
                                   summary_writer=writers[key])
        log.info("eval %s | step: %6d | metrics: %s", key, step, _fmt(m))
        metrics[_val_logdir(key)] = m

  def train(self, task: task_lib.Task) -> core.Logs:
    train_iter, _, state, train_step, _, step = self.process_task(task, training=True)
    log.info("train | step: %6d | training for %d steps...", step, self._train_steps)
    metrics: dict[str, Any] = {}
    while step < self._train_steps:
      n = min(self._train_steps - step, self._steps_per_loop)
      state, tm = self._train_n_steps(train_iter=train_iter, train_step=train_step, state=state,
                                      start_step=step, num_steps=n,
                                      summary_writer=self.train_summary_writer)
      curr = step + n - 1
      log.info("train | step: %6d | metrics: %s", curr, _fmt(tm))
      metrics[core.TRAIN_LOG_DIRNAME] = tm
      self._maybe_save_checkpoint(curr, state, metrics=metrics)
      step = curr + 1
    self._finish_training(task, state)
    return metrics

  def evaluate(self, task: task_lib.Task) -> core.Logs:
    _, eval_iters, state, _, eval_step, step = self.process_task(task, training=False)
    metrics: dict[str, Any] = {}
    self._run_evals(eval_iters, eval_step, state, step, self._eval_writers(eval_iters), metrics)
    return metrics

  def train_and_evaluate(self, task: task_lib.Task) -> core.Logs:
    train_iter, eval_iters, state, train_step, eval_step, step = self.process_task(
        task, training=True)
    writers = self._eval_writers(eval_iters)
    metrics: dict[str, Any] = {}
    while step < self._train_steps:
      n = min(self._train_steps - step, self._steps_per_loop)
      state, tm = self._train_n_steps(train_iter=train_iter, train_step=train_step, state=state,
                                      start_step=step, num_steps=n,
                                      summary_writer=self.train_summary_writer)
      curr = step + n - 1
      log.info("train | step: %6d | metrics: %s", curr, _fmt(tm))
      metrics[core.TRAIN_LOG_DIRNAME] = tm
      self._run_evals(eval_iters, eval_step, state, curr, writers, metrics)
      self._maybe_save_checkpoint(curr, state, metrics=metrics)
      step = curr + 1
    self._finish_training(task, state)
    return metrics

  def evaluate_continuously(self, task: task_lib.Task) -> core.Logs:
    _, eval_iters, state, _, eval_step, _ = self.process_task(
        task, training=False, check_for_checkpoints=False)
    writers = self._eval_writers(eval_iters)
    marker = os.path.join(self._model_dir, core.TRAINING_COMPLETE_MARKER_FILE)
    metrics: dict[str, Any] = {}
    for step in ckpt_lib.checkpoints_iterator(
        os.path.join(self._model_dir, core.CHECKPOINT_DIR),
        timeout=self._continuous_eval_timeout, timeout_fn=lambda: os.path.exists(marker)):
      try:
        state = self._maybe_restore_checkpoint(state, step)
        self._run_evals(eval_iters, eval_step, state, step, writers, metrics)
      except FileNotFoundError:
        log.info("Checkpoint step %s did not finish writing; skipping.", step)
    return metrics


JaxTrainer = Trainer
