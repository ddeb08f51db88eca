"""Host-side id preprocessing on the native library (`csrc/host/id_preprocess.cpp`): packing
per-feature id lists into a `KeyedJagged`, partitioning a table's ids by owning shard with duplicate
merging / dropping, and the per-partition statistics (max ids, max unique ids, drops) that the
reference records for buffer sizing (`SparseDenseMatmulInputStats`) and feeds back through its
file-based FDO client.  `ShardedPreprocessor` is the iterator post-processor that turns raw batches
into what `ShardedEmbedding` consumes (role of `SparsecorePreprocessor`,
`recml/layers/linen/sparsecore.py:272-354`)."""
from __future__ import annotations

import ctypes
import dataclasses
import os
from typing import Mapping, Sequence

import numpy as np
import torch

from recml_b200.embedding.jagged import KeyedJagged
from recml_b200.ops import _lib

c_ll, c_int = ctypes.c_longlong, ctypes.c_int


def pack_jagged(features: Mapping[str, Sequence[np.ndarray]], weights: Mapping[str, np.ndarray] | None = None,
                pin: bool = False) -> KeyedJagged:
  """`features[name] = (ids int64[nnz_f], lengths int32[batch])` → one KeyedJagged, built by all host threads."""
  lib = _lib.host()
  names = tuple(features)
  F = len(names)
  ids = [np.ascontiguousarray(features[n][0], dtype=np.int64) for n in names]
  lens = [np.ascontiguousarray(features[n][1], dtype=np.int32) for n in names]
  batch = int(lens[0].size) if F else 0
  for n, a, l in zip(names, ids, lens):       # the native packer trusts these
    if l.size != batch or (l.size and int(l.min()) < 0) or int(l.sum(dtype=np.int64)) != a.size:
      raise ValueError(f"feature {n!r}: {a.size} ids, lengths of {l.size} samples summing to "
                       f"{int(l.sum(dtype=np.int64))} (batch {batch})")
  total = int(sum(a.size for a in ids))
  mk = (lambda *s, dtype: torch.empty(*s, dtype=dtype).pin_memory()) if (pin and torch.cuda.is_available()) else \
      (lambda *s, dtype: torch.empty(*s, dtype=dtype))
  values, offsets = mk(total, dtype=torch.int32), mk(F * batch + 1, dtype=torch.int32)
  w_out = mk(total, dtype=torch.float32) if weights is not None else None
  P = ctypes.c_void_p
  id_ptrs = (P * F)(*[a.ctypes.data for a in ids])
  len_ptrs = (P * F)(*[a.ctypes.data for a in lens])
  w_ptrs = None
  if weights is not None:
    ws = [None if weights.get(n) is None else np.ascontiguousarray(weights[n], dtype=np.float32) for n in names]
    w_ptrs = (P * F)(*[0 if w is None else w.ctypes.data for w in ws])
  rc = lib.recml_pack_jagged(c_int(F), c_int(batch), id_ptrs, len_ptrs, w_ptrs, P(values.data_ptr()),
                             P(offsets.data_ptr()), P(0 if w_out is None else w_out.data_ptr()))
  if rc != 0:
    raise ValueError("batch holds more than 2^31 ids")
  return KeyedJagged(names, values, offsets, w_out, batch)


@dataclasses.dataclass
class PartitionStats:
  """Per-table statistics of one batch (`max_ids_per_partition`, `max_unique_ids_per_partition`, drops)."""
  max_ids_per_partition: int
  max_unique_ids_per_partition: int
  dropped_ids: int


def partition_csr(ids: np.ndarray, offsets: np.ndarray, shards: int, *, rotation: int = 0, gains: np.ndarray | None = None,
                  max_ids_per_partition: int = 0):
  """ids of one table (jagged by sample) → (rows, samples, gains, shard_ptr, stats): entries sorted by
  (shard, local row, sample), duplicate (row, sample) pairs merged by adding gains, at most
  `max_ids_per_partition` entries kept per shard (0 = unlimited)."""
  lib = _lib.host()
  lib.recml_partition_csr.restype = c_ll
  ids = np.ascontiguousarray(ids, dtype=np.int32)
  offsets = np.ascontiguousarray(offsets, dtype=np.int32)
  nnz, batch = int(offsets[-1]), offsets.size - 1
  rows, samples = np.empty(nnz, np.int32), np.empty(nnz, np.int32)
  out_g = np.empty(nnz, np.float32)
  ptr, stats = np.zeros(shards + 1, np.int64), np.zeros(3, np.int64)
  g = None if gains is None else np.ascontiguousarray(gains, dtype=np.float32)
  P = ctypes.c_void_p
  kept = lib.recml_partition_csr(P(ids.ctypes.data), P(offsets.ctypes.data), P(0 if g is None else g.ctypes.data),
                                 c_int(batch), c_int(shards), c_int(rotation), c_int(max_ids_per_partition),
                                 P(rows.ctypes.data), P(samples.ctypes.data), P(out_g.ctypes.data),
                                 P(ptr.ctypes.data), P(stats.ctypes.data))
  if kept == -1:
    raise ValueError("negative id in the batch")
  if kept < 0:
    raise ValueError(f"bad partition request: {shards} shards, offsets must ascend from 0")
  return rows[:kept], samples[:kept], out_g[:kept], ptr, PartitionStats(int(stats[0]), int(stats[1]), int(stats[2]))


class StatsRecorder:
  """Feedback-directed sizing: keeps the running maxima of the per-partition statistics per table and
  persists them as an `.npz` (the reference's file FDO client does the same per process)."""

  def __init__(self, base_dir: str | None = None, process_index: int = 0):
    self.base_dir, self.process_index = base_dir, process_index
    self.max_ids: dict[str, int] = {}
    self.max_unique: dict[str, int] = {}
    self.dropped: dict[str, int] = {}

  def record(self, table: str, stats: PartitionStats) -> None:
    self.max_ids[table] = max(self.max_ids.get(table, 0), stats.max_ids_per_partition)
    self.max_unique[table] = max(self.max_unique.get(table, 0), stats.max_unique_ids_per_partition)
    self.dropped[table] = self.dropped.get(table, 0) + stats.dropped_ids

  def _path(self) -> str:
    return os.path.join(self.base_dir, f"fdo_stats_{self.process_index}.npz")

  def publish(self) -> str:
    os.makedirs(self.base_dir, exist_ok=True)
    names = sorted(self.max_ids)
    np.savez(self._path(), tables=np.array(names), max_ids=np.array([self.max_ids[n] for n in names]),
             max_unique=np.array([self.max_unique[n] for n in names]),
             dropped=np.array([self.dropped[n] for n in names]))
    return self._path()

  def load(self) -> dict[str, PartitionStats]:
    """Maxima over the files of all processes found in `base_dir`."""
    out: dict[str, PartitionStats] = {}
    for f in sorted(os.listdir(self.base_dir)):
      if not (f.startswith("fdo_stats_") and f.endswith(".npz")):
        continue
      z = np.load(os.path.join(self.base_dir, f))
      for n, a, b, d in zip(z["tables"], z["max_ids"], z["max_unique"], z["dropped"]):
        prev = out.get(str(n), PartitionStats(0, 0, 0))
        out[str(n)] = PartitionStats(max(prev.max_ids_per_partition, int(a)),
                                     max(prev.max_unique_ids_per_partition, int(b)), prev.dropped_ids + int(d))
    return out


class ShardedPreprocessor:
  """Iterator post-processor: raw batch {feature: `[B, L]` ids or (ids, lengths)} → adds
  `batch[output_key]` = KeyedJagged in the embedding's feature order; optionally records statistics."""

  def __init__(self, feature_names: Sequence[str], *, output_key: str = "sparse", world: int = 1,
               table_of: Mapping[str, str] | None = None, recorder: StatsRecorder | None = None,
               max_ids_per_partition: int = 0, pin: bool = False):
    self.names, self.output_key, self.world = tuple(feature_names), output_key, world
    self.table_of = dict(table_of or {})
    self.recorder, self.cap, self.pin = recorder, max_ids_per_partition, pin

  def __call__(self, batch: dict) -> dict:
    feats = {}
    for n in self.names:
      x = batch[n]
      if isinstance(x, dict):
        feats[n] = (x["values"], x["lengths"])
      elif isinstance(x, tuple):
        feats[n] = x
      else:
        x = np.asarray(x)
        x = x[:, None] if x.ndim == 1 else x
        feats[n] = (x.reshape(-1), np.full(x.shape[0], x.shape[1], np.int32))
    kjt = pack_jagged(feats, pin=self.pin)
    if self.recorder is not None:
      for n in self.names:
        ids, lens = feats[n]
        offs = np.zeros(len(lens) + 1, np.int32)
        np.cumsum(lens, out=offs[1:])
        *_, stats = partition_csr(ids, offs, self.world, max_ids_per_partition=self.cap)
        self.recorder.record(self.table_of.get(n, n), stats)
    out = {k: v for k, v in batch.items() if k not in self.names}
    out[self.output_key] = kjt
    return out
