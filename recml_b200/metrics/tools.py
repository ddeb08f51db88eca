"""Metric logging: TensorBoard writer and the asynchronous accumulator
(`recml/core/metrics/tools.py:33-159`)."""
from __future__ import annotations

import concurrent.futures
import functools
import os
from typing import Any, Mapping

import numpy as np

from recml_b200.metrics import base


class AsyncMultiWriter:
  """Writes scalars to `<log_dir>/<name>` as TensorBoard events (and keeps the last
  values in memory for tests / logging)."""

  def __init__(self, *, log_dir: str, name: str):
    from torch.utils.tensorboard import SummaryWriter
    self._path = os.fspath(os.path.join(log_dir, name))
    os.makedirs(self._path, exist_ok=True)
    self._writer = SummaryWriter(self._path)
    self.last: dict[str, float] = {}

  @property
  def summary_writer(self) -> "AsyncMultiWriter":
    return self

  @property
  def log_path(self) -> str:
    return self._path

  def write_scalars(self, step: int, scalars: Mapping[str, Any]) -> None:
    for k, v in scalars.items():
      arr = np.asarray(v)
      if arr.size == 1:
        self._writer.add_scalar(k, float(arr.reshape(())), global_step=step)
        self.last[k] = float(arr.reshape(()))
      else:
        for i, x in enumerate(arr.reshape(-1)):
          self._writer.add_scalar(f"{k}/{i}", float(x), global_step=step)

  def flush(self) -> None:
    self._writer.flush()

  def close(self) -> None:
    self._writer.close()


def compute_metrics(metrics: Mapping[str, base.Metric]) -> dict[str, base.Scalar]:
  return {k: m.compute() for k, m in metrics.items()}


def merge_metrics(a: Mapping[str, base.Metric], b: Mapping[str, base.Metric]):
  out = dict(a)
  for k, v in b.items():
    out[k] = out[k].merge(v) if k in out else v
  return out


def _localize_all(ms: Mapping[str, base.Metric]) -> dict[str, base.Metric]:
  return {k: m.localize() for k, m in ms.items()}


def _log_step_scalars(writer, step, ms):
  writer.write_scalars(step, compute_metrics(_localize_all(ms)))


class MetricAccumulator:
  """Collects per-step metric states; per-step `ScalarMetric`s are pulled to the host
  and logged on a worker thread so the training loop never waits on a D2H copy; all
  other metrics are merged and written once per loop by `compute_and_log_scalars`."""

  def __init__(self, writer: AsyncMultiWriter, max_workers: int = 1,
               reduce_across_ranks: bool = False):
    if not isinstance(writer, AsyncMultiWriter):
      raise ValueError(f"`writer` must be an AsyncMultiWriter, got {type(writer)}.")
    self._writer = writer
    self._metrics: list[Mapping[str, base.Metric]] = []
    self._pool = concurrent.futures.ThreadPoolExecutor(max_workers=max_workers)
    self._futures: list[concurrent.futures.Future] = []
    self._reduce = reduce_across_ranks

  def accumulate(self, metrics: Mapping[str, base.Metric], step: int) -> None:
    self._metrics.append(metrics)
    scalars = {k: v for k, v in metrics.items() if isinstance(v, base.ScalarMetric)}
    if scalars:
      self._futures.append(self._pool.submit(_log_step_scalars, self._writer, step, scalars))

  def compute_and_log_scalars(self, step: int) -> dict[str, base.Scalar]:
    if not self._metrics:
      return {}
    for f in self._futures:
      f.result()
    self._futures.clear()
    if self._reduce:
      merged = functools.reduce(merge_metrics, self._metrics)
      merged = {k: m.reduce_across_ranks() for k, m in merged.items()}
      merged = _localize_all(merged)
    else:
      merged = functools.reduce(merge_metrics, [_localize_all(m) for m in self._metrics])
    self._metrics.clear()
    scalars = compute_metrics(merged)
    self._writer.write_scalars(
        step, {k: v for k, v in scalars.items() if not isinstance(merged[k], base.ScalarMetric)})
    self._writer.flush()
    return scalars
