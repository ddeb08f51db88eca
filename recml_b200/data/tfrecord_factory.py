"""Dataset factory over TFRecord files (`recml/core/data/tf_dataset_factory.py:214-583`): file
globbing, per-process file sharding, file / record shuffling, batching, `tf.Example` parsing by a
feature spec, preprocessors / postprocessors, label popping, a `debug` single cached batch, repeat
and a background prefetch thread that stages batches in pinned memory.  Field names follow the
reference where they are meaningful without tf.data."""
from __future__ import annotations

import dataclasses
import glob as glob_lib
import queue
import threading
from typing import Any, Callable, Mapping, Sequence

import numpy as np
import torch
import torch.distributed as dist

from recml_b200.data import iterator as iterator_lib
from recml_b200.data import tfrecord
from recml_b200.utils import types


@dataclasses.dataclass(frozen=True)
class DatasetShardingInfo:
  """Which slice of the input this process reads (`tf_dataset_factory.py:79-92`)."""
  num_processes: int = 1
  process_index: int = 0

  def per_process_batch_size(self, global_batch_size: int) -> int:
    if global_batch_size % self.num_processes:
      raise ValueError(f"global batch {global_batch_size} not divisible by {self.num_processes} processes")
    return global_batch_size // self.num_processes

  @classmethod
  def current(cls) -> "DatasetShardingInfo":
    if dist.is_available() and dist.is_initialized():
      return cls(dist.get_world_size(), dist.get_rank())
    return cls()


@dataclasses.dataclass(frozen=True)
class FixedLenFeature:
  shape: tuple[int, ...]
  dtype: str = "int64"
  default_value: Any = 0


@dataclasses.dataclass(frozen=True)
class VarLenFeature:
  dtype: str = "int64"


def get_file_groups(input_path: str | Sequence[str], sharding: DatasetShardingInfo) -> list[str]:
  """Expands glob(s) and keeps every `num_processes`-th file starting at `process_index`; with fewer
  files than processes every process reads all files (records are then sharded instead)."""
  pats = [input_path] if isinstance(input_path, str) else list(input_path)
  files = sorted(f for p in pats for f in glob_lib.glob(p))
  if not files:
    raise FileNotFoundError(f"No files match {pats}")
  if len(files) >= sharding.num_processes:
    return files[sharding.process_index::sharding.num_processes]
  return files


class _RecordDataset:
  def __init__(self, fac: "TFDatasetFactory"):
    self.fac = fac
    self.sharding = fac.sharding_info or DatasetShardingInfo.current()
    self.files = get_file_groups(fac.input_path, self.sharding)
    all_files = sorted(f for p in ([fac.input_path] if isinstance(fac.input_path, str) else fac.input_path)
                       for f in glob_lib.glob(p))
    self.shard_records = len(all_files) < self.sharding.num_processes
    self.batch = self.sharding.per_process_batch_size(fac.global_batch_size)
    self._cached = None

  def _parse(self, rf: tfrecord.RecordFile, rows: np.ndarray) -> dict:
    out = {}
    for name, spec in self.fac.feature_spec.items():
      if isinstance(spec, FixedLenFeature):
        n = int(np.prod(spec.shape)) if spec.shape else 1
        arr = rf.parse(rows, name, spec.dtype, n, spec.default_value).reshape((len(rows),) + tuple(spec.shape))
        out[name] = arr
      else:
        vals, lens = rf.parse(rows, name, spec.dtype)
        out[name] = {"values": vals, "lengths": lens}
    for fn in self.fac.preprocessors:
      out = fn(out)
    if self.fac.label_name is not None:
      label = out.pop(self.fac.label_name)
      out = (out, label)
    for fn in self.fac.postprocessors:
      out = fn(out)
    return out

  def _generate(self):
    fac = self.fac
    rng = np.random.default_rng(fac.seed)
    epoch = 0
    while True:
      files = list(self.files)
      if fac.file_shuffle:
        rng.shuffle(files)
      for path in files:
        rf = tfrecord.RecordFile(path, verify=fac.verify_checksums)
        rows = np.arange(len(rf))
        if self.shard_records:
          rows = rows[self.sharding.process_index::self.sharding.num_processes]
        if fac.shuffle:
          rng.shuffle(rows)
        for a in range(0, len(rows), self.batch):
          chunk = rows[a:a + self.batch]
          if len(chunk) < self.batch and fac.drop_remainder:
            continue
          yield self._parse(rf, chunk)
      epoch += 1
      if not fac.repeat or (fac.num_epochs is not None and epoch >= fac.num_epochs):
        return

  def __iter__(self):
    fac = self.fac
    if fac.debug:
      if self._cached is None:
        self._cached = next(self._generate())
      while True:
        yield self._cached
    if fac.prefetch_buffer_size <= 0:
      yield from self._generate()
      return
    q: "queue.Queue" = queue.Queue(maxsize=fac.prefetch_buffer_size)
    stop = threading.Event()

    def work():
      try:
        for b in self._generate():
          if stop.is_set():
            return
          q.put(("ok", b))
        q.put(("end", None))
      except BaseException as e:  # propagate loader failures to the consumer
        q.put(("err", e))

    th = threading.Thread(target=work, daemon=True, name="recml-tfrecord-prefetch")
    th.start()
    try:
      while True:
        kind, item = q.get()
        if kind == "end":
          return
        if kind == "err":
          raise item
        yield item
    finally:
      stop.set()


class TFDatasetFactory(types.Factory[iterator_lib.Iterator]):
  input_path: str | Sequence[str]
  feature_spec: Mapping[str, FixedLenFeature | VarLenFeature]
  global_batch_size: int
  drop_remainder: bool = True
  shuffle: bool = False
  file_shuffle: bool = False
  repeat: bool = False
  num_epochs: int | None = None
  seed: int = 0
  label_name: str | None = None
  preprocessors: Sequence[Callable[[Any], Any]] = ()
  postprocessors: Sequence[Callable[[Any], Any]] = ()
  prefetch_buffer_size: int = 2
  verify_checksums: bool = True
  debug: bool = False
  sharding_info: DatasetShardingInfo | None = None

  def make(self) -> iterator_lib.Iterator:
    return iterator_lib.IterableIterator(_RecordDataset(self))
