"""Dataset factory over TFRecord files (`recml/core/data/tf_dataset_factory.py:214-583`): file
globbing, per-process file sharding (or none), directory groups read newest first, file / record
shuffling, interleaved reading, batching, `tf.Example` / `tf.SequenceExample` parsing by a feature spec, a
vectorised filter with re-batching, preprocessor(s) / postprocessors, label popping, a `debug` single cached
batch, repeat (of the records or of the file list) and a background prefetch thread that stages batches in
pinned memory.  Field names follow the reference where they are meaningful without tf.data; its TFDS,
tf.Transform and tf.data-service hooks name external services and have no counterpart."""
from __future__ import annotations

import dataclasses
import enum
import functools
import glob as glob_lib
import queue
import threading
from typing import Any, Callable, Mapping, Sequence

import numpy as np
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


class FileFormat(enum.Enum):
  """Container formats the reference can read (`tf_dataset_factory.py:65-76`).  TFRecord is the one with a
  reader here; the others are Google-internal or need the array_record library."""
  TFRECORD = "tfrecord"
  RECORDIO = "recordio"
  SSTABLE = "sstable"
  ARRAY_RECORD = "array_record"


def expand_input_paths(input_path: str | Sequence[str]) -> list[str]:
  """All files matching the glob(s), sorted."""
  pats = [input_path] if isinstance(input_path, str) else list(input_path)
  files = sorted(f for p in pats for f in glob_lib.glob(p))
  if not files:
    raise FileNotFoundError(f"No input files found for patterns: {pats}.")
  return files


def get_file_groups(files: Sequence[str]) -> list[str]:
  """Groups files by their directory; every group is its paths joined by commas and the groups come in
  DESCENDING directory order, so that with `Span-<n>/...` layouts the newest span is read first
  (`tf_dataset_factory.py:809-868`)."""
  if not files:
    raise ValueError("`files` is empty.")
  groups: dict[str, list[str]] = {}
  for f in files:
    groups.setdefault(f[:f.rfind("/")], []).append(f)
  return [",".join(groups[d]) for d in sorted(groups, reverse=True)]


def _take(features: dict, idx: np.ndarray) -> dict:
  """Rows `idx` of a parsed feature dict (dense arrays and {"values", "lengths"[, "steps"]} jagged ones)."""
  out = {}
  for k, v in features.items():
    if isinstance(v, dict):
      lens = v["lengths"]
      starts = np.zeros(len(lens) + 1, dtype=np.int64)
      np.cumsum(lens, out=starts[1:])
      pieces = [v["values"][starts[i]:starts[i + 1]] for i in idx]
      item = {"values": np.concatenate(pieces) if pieces else v["values"][:0], "lengths": lens[idx]}
      if "steps" in v:
        item["steps"] = v["steps"][idx]
      out[k] = item
    else:
      out[k] = v[idx]
  return out


def _concat(parts: list[dict]) -> dict:
  out = {}
  for k, v in parts[0].items():
    if isinstance(v, dict):
      out[k] = {kk: np.concatenate([p[k][kk] for p in parts]) for kk in v}
    else:
      out[k] = np.concatenate([p[k] for p in parts])
  return out


def _rows_of(features: dict) -> int:
  v = next(iter(features.values()))
  return len(v["lengths"]) if isinstance(v, dict) else len(v)


class _RecordDataset:
  def __init__(self, fac: "TFDatasetFactory"):
    self.fac = fac
    if fac.file_format not in (FileFormat.TFRECORD, "tfrecord"):
      raise ValueError(f"File format: {fac.file_format} is not supported. Expected one of: {[FileFormat.TFRECORD]}.")
    self.sharding = fac.sharding_info or DatasetShardingInfo.current()
    # A reading unit is one file, or with `group_uris_by_dir` all files of one directory read one after the
    # other.  Units (not records) are what gets shuffled, sharded over processes and interleaved; with fewer
    # units than processes every process opens all of them and takes every n-th record instead.
    files = fac.input_filepaths
    groups = [g.split(",") for g in get_file_groups(files)] if fac.group_uris_by_dir else [[f] for f in files]
    self.files = [f for g in groups for f in g]
    at = 0
    self.units: list[list[int]] = []
    for g in groups:
      self.units.append(list(range(at, at + len(g))))
      at += len(g)
    shard = fac.sharding and self.sharding.num_processes > 1
    self.shard_records = shard and len(self.units) < self.sharding.num_processes
    self.shard_units = shard and not self.shard_records
    self.batch = self.sharding.per_process_batch_size(fac.global_batch_size)
    self._cached = None

  def _units_of_epoch(self, epoch: int) -> list[int]:
    ids = list(range(len(self.units)))
    if not self.shard_units:
      return ids
    n, p = self.sharding.num_processes, self.sharding.process_index
    if self.fac.repeat and self.fac.repeat_files:
      # the unit list is repeated BEFORE it is dealt out, so a process sees other units in the next pass
      # unless the number of units is a multiple of the number of processes
      base = epoch * len(ids)
      return [i for i in ids if (base + i) % n == p]
    return ids[p::n]

  def _parse_features(self, rf: tfrecord.RecordFile, rows: np.ndarray) -> dict:
    out = {}
    # every tf.Example feature in one pass over each record
    specs = []
    for name, spec in self.fac.feature_spec.items():
      if isinstance(spec, FixedLenFeature):
        specs.append((name, spec.dtype, int(np.prod(spec.shape)) if spec.shape else 1, spec.default_value))
      else:
        specs.append((name, spec.dtype, 0, 0))
    seq = self.fac.sequence_feature_spec or {}
    one_call = not (set(seq) & set(self.fac.feature_spec))       # results are keyed by name
    if one_call:
      specs += [(name, spec.dtype, 0, 0, "list") for name, spec in seq.items()]   # tf.SequenceExample feature lists
    parsed = rf.parse_many(rows, specs) if specs else {}
    for name, spec in self.fac.feature_spec.items():
      if isinstance(spec, FixedLenFeature):
        out[name] = parsed[name].reshape((len(rows),) + tuple(spec.shape))
      else:
        vals, lens = parsed[name]
        out[name] = {"values": vals, "lengths": lens}
    for name, spec in seq.items():
      vals, lens, steps = parsed[name] if one_call else rf.parse_sequence(rows, name, spec.dtype)
      out[name] = {"values": vals, "lengths": lens, "steps": steps}
    return out

  def _finish(self, out: dict):
    if self.fac.preprocessor is not None:
      out = self.fac.preprocessor(out)
    for fn in self.fac.preprocessors:
      out = fn(out)
    if self.fac.label_name is not None:
      label = out.pop(self.fac.label_name)
      out = (out, label)
    for fn in self.fac.postprocessors:
      out = fn(out)
    return out

  def _record_stream(self, rng, epoch: int = 0):
    """(file indices, record indices) array pairs in reading order: `cycle_length` files are open at a time
    and `block_length` records are taken from each in turn (tf.data `interleave`); then an optional shuffle
    window.  The order is produced in blocks with numpy, not record by record."""
    fac = self.fac
    units = self._units_of_epoch(epoch)
    if fac.file_shuffle:
      rng.shuffle(units)

    def rows_of(ui):
      """(file index, record index) of every record of a unit, in reading order."""
      fs, rs = [], []
      for fi in self.units[ui]:
        n = len(self._open(fi))
        rows = np.arange(n, dtype=np.int64)
        if self.shard_records:
          rows = rows[self.sharding.process_index::self.sharding.num_processes]
        if fac.shuffle and not fac.shuffle_buffer_size:
          rng.shuffle(rows)
        fs.append(np.full(len(rows), fi, dtype=np.int64))
        rs.append(rows)
      return (np.concatenate(fs), np.concatenate(rs)) if len(fs) > 1 else (fs[0], rs[0])

    def interleaved():
      cycle = max(1, fac.cycle_length or 1)
      blk = max(1, fac.block_length)
      pending = list(units)
      active: list[tuple[np.ndarray, np.ndarray, int]] = []       # (file indices, record indices, position)
      while pending or active:
        while pending and len(active) < cycle:
          active.append((*rows_of(pending.pop(0)), 0))
        active = [a for a in active if a[2] < len(a[1])]
        if not active:
          continue
        if len(active) == 1 and (cycle == 1 or not pending):
          fs, rows, at = active[0]                  # one open unit: its blocks follow one another anyway
          yield fs[at:], rows[at:]
          active = []
          continue
        # whole rounds (one block from every open unit) until the first unit runs short of a full block
        k = min((len(rows) - at) // blk for _, rows, at in active)
        if k >= 1:
          parts_r = np.stack([rows[at:at + k * blk].reshape(k, blk) for _, rows, at in active], axis=1)
          parts_f = np.stack([fs[at:at + k * blk].reshape(k, blk) for fs, _, at in active], axis=1)
          yield parts_f.reshape(-1), parts_r.reshape(-1)
          active = [(fs, rows, at + k * blk) for fs, rows, at in active]
          continue
        nxt = []                                   # a round with a short last block
        for fs, rows, at in active:
          hi = min(at + blk, len(rows))
          yield fs[at:hi], rows[at:hi]
          if hi < len(rows):
            nxt.append((fs, rows, hi))
        active = nxt

    if not (fac.shuffle and fac.shuffle_buffer_size):
      yield from interleaved()
      return
    # shuffle window: keep up to shuffle_buffer_size - 1 records back, emit the surplus in random order
    keep = max(0, int(fac.shuffle_buffer_size) - 1)
    win_f, win_r = np.zeros(0, np.int64), np.zeros(0, np.int64)
    for bf, br in interleaved():
      win_f, win_r = np.concatenate([win_f, bf]), np.concatenate([win_r, br])
      n_out = len(win_r) - keep
      if n_out > 0:
        perm = rng.permutation(len(win_r))
        out, rest = perm[:n_out], perm[n_out:]
        yield win_f[out], win_r[out]
        win_f, win_r = win_f[rest], win_r[rest]
    if len(win_r):
      perm = rng.permutation(len(win_r))
      yield win_f[perm], win_r[perm]

  def _open(self, fi: int) -> tfrecord.RecordFile:
    if fi not in self._open_cache:
      if not self.fac.cache_reading and len(self._open_cache) > 2 * max(1, self.fac.cycle_length or 1) + 2:
        self._open_cache.clear()          # `cache_reading` keeps every file (mapping and record index) open
      self._open_cache[fi] = tfrecord.RecordFile(self.files[fi], verify=self.fac.verify_checksums)
    return self._open_cache[fi]

  def _parse_mixed(self, fis: np.ndarray, rows: np.ndarray) -> dict:
    """Parses records that may come from several files, keeping the given order."""
    uniq = list(dict.fromkeys(fis.tolist())) if len(fis) and (fis != fis[0]).any() else [int(fis[0])]
    if len(uniq) == 1:
      return self._parse_features(self._open(uniq[0]), rows)
    parts, order = [], []
    for fi in uniq:
      sel = np.nonzero(fis == fi)[0]
      parts.append(self._parse_features(self._open(fi), rows[sel]))
      order.append(sel)
    merged = _concat(parts)
    inv = np.argsort(np.concatenate(order), kind="stable")
    return _take(merged, inv)

  def _batches_of(self, stream):
    """Cuts the stream of (file indices, record indices) blocks into pieces of the batch size; the last
    piece of an epoch may be shorter."""
    pend_f, pend_r, n = [], [], 0
    for bf, br in stream:
      pend_f.append(bf); pend_r.append(br); n += len(br)
      if n < self.batch:
        continue
      f, r = np.concatenate(pend_f), np.concatenate(pend_r)
      at = 0
      while n - at >= self.batch:
        yield f[at:at + self.batch], r[at:at + self.batch]
        at += self.batch
      pend_f, pend_r, n = ([f[at:]], [r[at:]], n - at) if at < n else ([], [], 0)
    if n:
      yield np.concatenate(pend_f), np.concatenate(pend_r)

  def _generate(self):
    fac = self.fac
    rng = np.random.default_rng(fac.seed)
    self._open_cache: dict = {}
    carry: list[dict] = []          # rows that passed the filter but do not fill a batch yet
    carried = 0

    def epochs():
      """The record stream of every epoch, one after the other: with `repeat` the records are repeated
      BEFORE batching (the reference repeats its file list), so batches run across epoch boundaries and
      an input smaller than one batch still fills batches."""
      epoch = 0
      while True:
        seen = 0
        for bf, br in self._record_stream(rng, epoch):
          seen += len(br)
          yield bf, br
        epoch += 1
        if seen == 0 or not fac.repeat or (fac.num_epochs is not None and epoch >= fac.num_epochs):
          return

    for fis, rows in self._batches_of(epochs()):
      if len(rows) < self.batch and fac.drop_remainder and fac.filter_fn is None:
        break
      feats = self._parse_mixed(fis, rows)
      if fac.filter_fn is None:
        yield self._finish(feats)
        continue
      keep = np.nonzero(np.asarray(fac.filter_fn(feats), dtype=bool))[0]   # vectorised filter, then re-batch
      if len(keep):
        carry.append(_take(feats, keep))
        carried += len(keep)
      while carried >= self.batch:
        merged = _concat(carry)
        yield self._finish(_take(merged, np.arange(self.batch)))
        rest = _rows_of(merged) - self.batch
        carry = [_take(merged, np.arange(self.batch, self.batch + rest))] if rest else []
        carried = rest
    if carried and not fac.drop_remainder:
      yield self._finish(_concat(carry))

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
  sequence_feature_spec: Mapping[str, VarLenFeature] | None = None   # feature lists of tf.SequenceExample records
  filter_fn: Callable[[dict], Any] | None = None   # parsed batch -> boolean keep mask; survivors are re-batched
  shuffle_buffer_size: int = 0                     # > 0: shuffle records in a window instead of per file
  cycle_length: int | None = None                  # files read concurrently (interleave)
  block_length: int = 1                            # consecutive records taken from a file per turn
  file_format: FileFormat = FileFormat.TFRECORD
  sharding: bool = True                            # False: every process reads the whole input
  group_uris_by_dir: bool = False                  # read, shard and interleave whole directories, newest first
  repeat_files: bool = False                       # with `repeat`: repeat the file list before it is sharded
  cache_reading: bool = False                      # keep every input file mapped and indexed between passes
  preprocessor: Callable[[Any], Any] | None = None  # applied before `preprocessors`

  @functools.cached_property
  def input_filepaths(self) -> Sequence[str]:
    """The input files (`tf_dataset_factory.py:326-353`)."""
    if not self.input_path:
      raise ValueError("`input_path` must be set.")
    return expand_input_paths(self.input_path)

  def make(self) -> iterator_lib.Iterator:
    return iterator_lib.IterableIterator(_RecordDataset(self))
