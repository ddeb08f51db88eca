"""Criteo-1TB input pipeline for the standalone DLRM-DCNv2 trainer.

File format (`recml/inference/models/jax/DLRM_DCNv2/dataloader.py:130-215`): every TFRecord is ONE
PRE-BATCHED tf.Example of `B` samples with
  `clicked`                      int64   [B]
  `int-feature-1` .. `-13`       float32 [B]
  `categorical-feature-14`..`-39` bytes  [B], string i = the raw little-endian int64 ids of sample
                                          i's bag (`decode_raw`), `multi_hot_sizes[f]` ids each.
Files are sharded over processes (`dataset.shard(process_count, process_index)`); training repeats
for ever and shuffles records in a window, evaluation is padded with zero-weight batches so that
every process runs the same number of steps.

`CriteoDataLoader` turns records into the framework's batch dict (`dense` [B,13], `sparse`
KeyedJagged, `label` [B], plus `weight` [B] in eval), parsing with the native reader on all host
threads.  `ThreadedProducer` is the bounded-queue producer of `dlrm_main.py:174-291` (worker
threads do parsing and id packing off the training thread).  `dummy_batch` is the cached random
batch of `dataloader.py:38-79`.
"""
from __future__ import annotations

import ctypes
import glob as glob_lib
import queue
import threading
from typing import Any, Callable, Iterator, Sequence

import numpy as np
import torch

from recml_b200.data import synthetic
from recml_b200.data import tfrecord
from recml_b200.embedding.jagged import KeyedJagged

LABEL = "clicked"
DENSE = tuple(f"int-feature-{i}" for i in range(1, 14))
SPARSE = tuple(f"categorical-feature-{i}" for i in range(14, 40))


def dummy_batch(batch_size: int, multi_hot_sizes: Sequence[int], vocab_sizes: Sequence[int], seed: int = 0) -> dict:
  """Uniform random batch: labels randint(0,2), dense U(0,0.9), ids uniform in [0, V)."""
  rng = np.random.default_rng(seed)
  ids = [rng.integers(0, v, size=(batch_size, m), dtype=np.int64) for v, m in zip(vocab_sizes, multi_hot_sizes)]
  return assemble(rng.integers(0, 2, batch_size).astype(np.float32),
                  rng.uniform(0.0, 0.9, (batch_size, len(DENSE))).astype(np.float32), ids)


def assemble(labels: np.ndarray, dense: np.ndarray, ids: Sequence[np.ndarray], weight: np.ndarray | None = None,
             names: Sequence[str] | None = None) -> dict:
  """Per-feature `[B, bag]` id matrices → the batch dict with one feature-major KeyedJagged."""
  B = labels.shape[0]
  names = tuple(names) if names is not None else tuple(f"cat_{i}" for i in range(len(ids)))
  lens = np.concatenate([np.full(B, a.shape[1], dtype=np.int64) for a in ids])
  offsets = np.zeros(lens.size + 1, dtype=np.int32)
  offsets[1:] = np.cumsum(lens)
  values = np.concatenate([a.reshape(-1) for a in ids]).astype(np.int32)
  out = {"dense": torch.from_numpy(np.ascontiguousarray(dense, dtype=np.float32)),
         "sparse": KeyedJagged(names, torch.from_numpy(values), torch.from_numpy(offsets), None, B),
         "label": torch.from_numpy(np.ascontiguousarray(labels, dtype=np.float32))}
  if weight is not None:
    out["weight"] = torch.from_numpy(np.ascontiguousarray(weight, dtype=np.float32))
  return out


def encode_record(labels: np.ndarray, dense: np.ndarray, ids: Sequence[np.ndarray]) -> bytes:
  """One pre-batched record in the reference's format (used by tests and export tools)."""
  feats: dict[str, Any] = {LABEL: [int(x) for x in labels]}
  for j, name in enumerate(DENSE):
    feats[name] = [float(x) for x in dense[:, j]]
  for f, name in enumerate(SPARSE[:len(ids)]):
    feats[name] = [np.ascontiguousarray(row, dtype="<i8").tobytes() for row in ids[f]]
  return tfrecord.encode_example(feats)


class CriteoDataLoader:
  """Iterable over batch dicts read from pre-batched Criteo TFRecords.

  batch_size is the per-record (= per-process) batch; records whose batch differs are rejected.
  `is_training` repeats for ever and shuffles within `shuffle_buffer` records; evaluation makes one
  pass and, when `eval_steps` is given, pads with zero-weight batches up to that many steps
  (`dataloader.py:262-288`).  Ids are taken modulo the vocabulary like the reference model does."""

  def __init__(self, file_pattern: str | Sequence[str], batch_size: int, *, vocab_sizes: Sequence[int],
               multi_hot_sizes: Sequence[int], is_training: bool = True, process_index: int = 0,
               process_count: int = 1, shuffle_buffer: int = 256, eval_steps: int | None = None, seed: int = 0,
               verify_crc: bool = False):
    pats = [file_pattern] if isinstance(file_pattern, str) else list(file_pattern)
    files = sorted(f for p in pats for f in glob_lib.glob(p))
    if not files:
      raise FileNotFoundError(f"no files match {file_pattern!r}")
    self.files = files[process_index::process_count]
    if not self.files:
      raise ValueError(f"{len(files)} files cannot be split over {process_count} processes")
    self.batch_size, self.vocab_sizes, self.multi_hot = batch_size, list(vocab_sizes), list(multi_hot_sizes)
    self.is_training, self.shuffle_buffer, self.eval_steps = is_training, shuffle_buffer, eval_steps
    self.verify_crc = verify_crc
    self._rng = np.random.default_rng(seed + process_index)
    self._offsets = None

  def _parse(self, rf: tfrecord.RecordFile, rows: np.ndarray) -> list[dict]:
    """Label and the 13 dense features in one pass over each record; the id features are decoded by the
    native library straight into the int32 feature-major value layout (modulo the vocabulary included)."""
    B, R, F = self.batch_size, len(rows), len(self.multi_hot)
    fixed = rf.parse_many(rows, [(LABEL, "int64", B, -1)] + [(n, "float", B, 0.0) for n in DENSE])
    labels = fixed[LABEL]
    if (labels[:, -1] < 0).any():
      raise ValueError(f"a record holds fewer than batch_size={B} samples")
    dense = np.stack([fixed[n] for n in DENSE], axis=-1)      # [R, B, 13]
    lib = tfrecord._lib_host()
    offs = np.ascontiguousarray(rf.offsets[rows])
    lens = np.ascontiguousarray(rf.lengths[rows])
    names = SPARSE[:F]
    total = B * int(sum(self.multi_hot))
    values = np.empty((R, total), dtype=np.int32)
    bad = lib.recml_decode_multihot_records(
        rf.data.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p), lens.ctypes.data_as(ctypes.c_void_p),
        ctypes.c_longlong(R), ctypes.c_int(F), (ctypes.c_char_p * F)(*[n.encode() for n in names]),
        (ctypes.c_int * F)(*self.multi_hot), (ctypes.c_longlong * F)(*self.vocab_sizes[:F]), ctypes.c_int(B),
        values.ctypes.data_as(ctypes.c_void_p))
    if bad:
      raise ValueError(f"{bad} (record, feature) pairs do not hold {B} bags of the configured multi-hot sizes")
    if self._offsets is None:       # the bag sizes are fixed, so every batch has the same offsets
      lens_all = np.concatenate([np.full(B, m, dtype=np.int64) for m in self.multi_hot])
      self._offsets = np.zeros(lens_all.size + 1, dtype=np.int32)
      self._offsets[1:] = np.cumsum(lens_all)
    keys = tuple(f"cat_{i}" for i in range(F))      # the names `assemble` gives the features
    out = []
    for r in range(R):
      item = {"dense": torch.from_numpy(np.ascontiguousarray(dense[r], dtype=np.float32)),
              "sparse": KeyedJagged(keys, torch.from_numpy(values[r]), torch.from_numpy(self._offsets), None, B),
              "label": torch.from_numpy(labels[r].astype(np.float32))}
      if not self.is_training:
        item["weight"] = torch.ones(B, dtype=torch.float32)
      out.append(item)
    return out

  def _records(self) -> Iterator[dict]:
    while True:
      order = self._rng.permutation(len(self.files)) if self.is_training else np.arange(len(self.files))
      seen = 0
      for fi in order:
        rf = tfrecord.RecordFile(self.files[fi], verify=self.verify_crc)
        n = len(rf)
        seen += n
        for lo in range(0, n, 16):
          yield from self._parse(rf, np.arange(lo, min(lo + 16, n)))
      if not self.is_training:
        return
      if seen == 0:
        raise ValueError(f"no records in {self.files}: a training loader would repeat nothing for ever")

  def __iter__(self) -> Iterator[dict]:
    if self.is_training:
      window: list[dict] = []
      for rec in self._records():
        if self.shuffle_buffer <= 1:
          yield rec
          continue
        window.append(rec)
        if len(window) >= self.shuffle_buffer:
          yield window.pop(int(self._rng.integers(len(window))))
      return
    n = 0
    for rec in self._records():
      if self.eval_steps is not None and n >= self.eval_steps:
        return
      yield rec
      n += 1
    if self.eval_steps is not None and n < self.eval_steps:
      B = self.batch_size
      pad = assemble(np.zeros(B, np.float32), np.zeros((B, len(DENSE)), np.float32),
                     [np.zeros((B, m), np.int64) for m in self.multi_hot], weight=np.zeros(B, np.float32))
      for _ in range(self.eval_steps - n):
        yield pad


class ThreadedProducer:
  """Runs `transform(item)` for the items of `source` on `num_workers` threads and hands results
  out in order through a bounded queue (`dlrm_main.py:174-291`: 16 workers, depth 256).  The
  training thread only dequeues; parsing, id packing and pinning happen on the workers."""

  _END = object()

  def __init__(self, source, transform: Callable[[Any], Any] | None = None, *, num_workers: int = 16,
               depth: int = 256, pin: bool = False):
    self._source, self._transform = source, transform
    self._workers, self._depth, self._pin = max(1, num_workers), max(1, depth), pin

  def _prepare(self, item):
    if self._transform is not None:
      item = self._transform(item)
    if self._pin and torch.cuda.is_available():
      item = {k: (v.pin_memory() if hasattr(v, "pin_memory") else v) for k, v in item.items()}
    return item

  def __iter__(self):
    from concurrent.futures import ThreadPoolExecutor
    out: queue.Queue = queue.Queue(self._depth)
    stop = threading.Event()

    def feed():
      try:
        with ThreadPoolExecutor(self._workers) as pool:
          pending: list = []
          for item in self._source:
            if stop.is_set():
              break
            pending.append(pool.submit(self._prepare, item))
            while len(pending) >= self._workers * 2:
              out.put(pending.pop(0).result())
          for fut in pending:
            out.put(fut.result())
        out.put(self._END)
      except BaseException as e:  # pylint: disable=broad-except
        out.put(e)

    t = threading.Thread(target=feed, daemon=True, name="recml-producer")
    t.start()
    try:
      while True:
        item = out.get()
        if item is self._END:
          return
        if isinstance(item, BaseException):
          raise item
        yield item
    finally:
      stop.set()
      while t.is_alive():          # unblock a producer waiting on a full queue
        try:
          out.get_nowait()
        except queue.Empty:
          t.join(0.01)


def synthetic_loader(batch_size: int, vocab_sizes, multi_hot_sizes, *, steps: int | None = None, seed: int = 0,
                     rank: int = 0, num_batches: int = 4):
  """Zipf / log-normal batches of the benchmark's shape, for runs without files."""
  return synthetic.SyntheticDLRMDataset(batch_size, vocab_sizes, multi_hot_sizes, num_batches=num_batches, seed=seed,
                                        rank=rank, steps=steps)
