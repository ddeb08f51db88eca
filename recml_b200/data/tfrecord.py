"""TFRecord / tf.Example I/O on the native reader (`csrc/data/tfrecord.cpp`), with a pure-Python
serializer for writing test and export files.  No TensorFlow involved."""
from __future__ import annotations

import ctypes
import os
import struct
from typing import Iterable, Mapping, Sequence

import numpy as np

from recml_b200.ops import _lib

c_ll = ctypes.c_longlong


def _lib_host():
  lib = _lib.host()
  lib.recml_tfrecord_index.restype = c_ll
  lib.recml_tfrecord_frame.restype = c_ll
  lib.recml_crc32c.restype = ctypes.c_uint32
  return lib


def crc32c(data: bytes) -> int:
  return int(_lib_host().recml_crc32c(data, c_ll(len(data))))


# ---- protobuf wire-format writer for tf.train.Example -------------------------------------------------
def _varint(v: int) -> bytes:
  v &= (1 << 64) - 1
  out = bytearray()
  while True:
    b = v & 0x7F
    v >>= 7
    out.append(b | (0x80 if v else 0))
    if not v:
      return bytes(out)


def _ld(num: int, payload: bytes) -> bytes:
  return _varint((num << 3) | 2) + _varint(len(payload)) + payload


def encode_example(features: Mapping[str, Sequence]) -> bytes:
  """Serialises {name: list of ints | floats | bytes} as a tf.train.Example."""
  entries = b""
  for name, vals in features.items():
    vals = list(vals) if not isinstance(vals, (bytes, str)) else [vals]
    if vals and isinstance(vals[0], (bytes, str)):
      body = b"".join(_ld(1, v if isinstance(v, bytes) else v.encode()) for v in vals)
      feat = _ld(1, body)
    elif vals and isinstance(vals[0], (float, np.floating)):
      feat = _ld(2, _ld(1, struct.pack(f"<{len(vals)}f", *vals)))
    else:
      feat = _ld(3, _ld(1, b"".join(_varint(int(v)) for v in vals)))
    entries += _ld(1, _ld(1, name.encode()) + _ld(2, feat))
  return _ld(1, entries)


def write_tfrecord(path: str, records: Iterable[bytes]) -> int:
  lib = _lib_host()
  n = 0
  with open(path, "wb") as f:
    for rec in records:
      buf = ctypes.create_string_buffer(len(rec) + 16)
      w = lib.recml_tfrecord_frame(rec, c_ll(len(rec)), buf)
      f.write(buf.raw[:w])
      n += 1
  return n


class RecordFile:
  """A TFRecord file mapped into memory and indexed (payload offsets / lengths); CRCs verified.  The parse
  methods raise `ValueError` for a record that does not decode as a `tf.Example` / `tf.SequenceExample` to its
  last byte (a field running past the record, a truncated packed list), as TensorFlow's parser does."""

  def __init__(self, path: str, verify: bool = True):
    self.path = path
    # mapped, not read: only the pages of the records a process parses are brought in
    self.data = (np.memmap(path, dtype=np.uint8, mode="r") if os.path.getsize(path) > 0
                 else np.zeros(0, dtype=np.uint8))
    lib = _lib_host()
    ptr = self.data.ctypes.data_as(ctypes.c_void_p)
    n = lib.recml_tfrecord_index(ptr, c_ll(self.data.size), None, None, c_ll(0), ctypes.c_int(int(verify)))
    if n < 0:
      raise IOError(f"{path}: corrupt TFRecord at record {-n - 1}")
    self.offsets = np.zeros(n, dtype=np.int64)
    self.lengths = np.zeros(n, dtype=np.int64)
    lib.recml_tfrecord_index(ptr, c_ll(self.data.size), self.offsets.ctypes.data_as(ctypes.c_void_p),
                             self.lengths.ctypes.data_as(ctypes.c_void_p), c_ll(n), ctypes.c_int(0))

  def __len__(self) -> int:
    return int(self.offsets.size)

  def record(self, i: int) -> bytes:
    return self.data[self.offsets[i]:self.offsets[i] + self.lengths[i]].tobytes()

  def _malformed(self, rows: np.ndarray, k: int) -> ValueError:
    return ValueError(f"{self.path}: record {int(np.asarray(rows)[k])} is not a valid serialized example")

  def validate(self, rows: np.ndarray) -> None:
    """Structural check of the given records (every nested message decodes to its end); a record is checked
    once, however many per-feature parses ask for it."""
    rows = np.asarray(rows, dtype=np.int64)
    if getattr(self, "_checked", None) is None:
      self._checked = np.zeros(len(self), dtype=bool)
    todo = rows[~self._checked[rows]]
    if todo.size == 0:
      return
    lib = _lib_host()
    lib.recml_validate_examples.restype = c_ll
    offs = np.ascontiguousarray(self.offsets[todo])
    lens = np.ascontiguousarray(self.lengths[todo])
    k = lib.recml_validate_examples(self.data.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p),
                                    lens.ctypes.data_as(ctypes.c_void_p), c_ll(len(todo)))
    if k >= 0:
      raise self._malformed(todo, k)
    self._checked[todo] = True

  def parse(self, rows: np.ndarray, name: str, dtype: str, fixed_len: int = 0, default=0):
    """Parses feature `name` of the given record indices with all host threads.
    fixed_len > 0 → dense `[len(rows), fixed_len]`; else (values, row_lengths) jagged."""
    lib = _lib_host()
    self.validate(rows)
    kind = 0 if dtype in ("int64", "int") else 1
    np_dt = np.int64 if kind == 0 else np.float32
    offs = np.ascontiguousarray(self.offsets[rows])
    lens = np.ascontiguousarray(self.lengths[rows])
    n = len(rows)
    args = (self.data.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p),
            lens.ctypes.data_as(ctypes.c_void_p), c_ll(n), name.encode(), ctypes.c_int(kind))
    di, df = c_ll(int(default) if kind == 0 else 0), ctypes.c_float(float(default) if kind == 1 else 0.0)
    if fixed_len > 0:
      out = np.empty((n, fixed_len), dtype=np_dt)
      lib.recml_parse_examples(*args, ctypes.c_int(fixed_len), di, df, out.ctypes.data_as(ctypes.c_void_p), None, None)
      return out
    row_len = np.zeros(n, dtype=np.int64)
    lib.recml_parse_examples(*args, ctypes.c_int(0), di, df, None, row_len.ctypes.data_as(ctypes.c_void_p), None)
    starts = np.zeros(n, dtype=np.int64)
    np.cumsum(row_len[:-1], out=starts[1:])
    vals = np.empty(int(row_len.sum()), dtype=np_dt)
    lib.recml_parse_examples(*args, ctypes.c_int(0), di, df, vals.ctypes.data_as(ctypes.c_void_p), None,
                             starts.ctypes.data_as(ctypes.c_void_p))
    return vals, row_len


  def parse_many(self, rows: np.ndarray, specs: Sequence[tuple]) -> dict:
    """Parses several features of the given records in ONE pass over each record (the per-feature
    `parse` walks a record's feature map once per call).  `specs`: (name, dtype, fixed_len, default)
    tuples, fixed_len 0 for variable length; a fifth element "list" marks a feature LIST of a
    tf.SequenceExample (variable length).  Returns name -> dense `[n, fixed_len]` array,
    (values, row_lengths) for variable-length features, (values, row_lengths, steps) for feature lists."""
    lib = _lib_host()
    is_list = [len(sp) > 4 and sp[4] == "list" for sp in specs]
    specs = [tuple(sp[:4]) for sp in specs]
    n, F = len(rows), len(specs)
    offs = np.ascontiguousarray(self.offsets[rows])
    lens = np.ascontiguousarray(self.lengths[rows])
    kinds = [0 if dt in ("int64", "int") else 1 for _, dt, _, _ in specs]
    names = (ctypes.c_char_p * F)(*[nm.encode() for nm, _, _, _ in specs])
    c_kinds = (ctypes.c_int * F)(*kinds)
    c_fixed = (ctypes.c_int * F)(*[int(fl) for _, _, fl, _ in specs])
    c_di = (c_ll * F)(*[int(d) if k == 0 else 0 for (_, _, _, d), k in zip(specs, kinds)])
    c_df = (ctypes.c_float * F)(*[float(d) if k == 1 else 0.0 for (_, _, _, d), k in zip(specs, kinds)])
    dense, rowlen, steps = {}, {}, {}
    c_dense, c_rows, c_steps = (ctypes.c_void_p * F)(), (ctypes.c_void_p * F)(), (ctypes.c_void_p * F)()
    c_src = (ctypes.c_int * F)(*[int(x) for x in is_list])
    for f, ((nm, _, fl, _), k) in enumerate(zip(specs, kinds)):
      if is_list[f]:
        if fl > 0:
          raise ValueError(f"feature list {nm!r} must be variable length")
        steps[f] = np.zeros(n, dtype=np.int64)
        c_steps[f] = steps[f].ctypes.data
      if fl > 0:
        dense[f] = np.empty((n, fl), dtype=np.int64 if k == 0 else np.float32)
        c_dense[f] = dense[f].ctypes.data
      else:
        rowlen[f] = np.zeros(n, dtype=np.int64)
        c_rows[f] = rowlen[f].ctypes.data
    lib.recml_parse_multi.restype = ctypes.c_void_p
    lib.recml_parse_multi_size.restype = c_ll
    handle = ctypes.c_void_p(lib.recml_parse_multi(
        self.data.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p),
        lens.ctypes.data_as(ctypes.c_void_p), c_ll(n), ctypes.c_int(F), names, c_kinds, c_fixed, c_di, c_df,
        c_dense, c_rows, c_src, c_steps))
    out = {}
    try:
      lib.recml_parse_multi_first_bad.restype = c_ll
      bad = lib.recml_parse_multi_first_bad(handle)
      if bad >= 0:
        raise self._malformed(rows, bad)
      for f, ((nm, _, fl, _), k) in enumerate(zip(specs, kinds)):
        if fl > 0:
          out[nm] = dense[f]
          continue
        vals = np.empty(int(lib.recml_parse_multi_size(handle, ctypes.c_int(f))), dtype=np.int64 if k == 0 else np.float32)
        lib.recml_parse_multi_fetch(handle, ctypes.c_int(f), vals.ctypes.data_as(ctypes.c_void_p))
        out[nm] = (vals, rowlen[f], steps[f]) if is_list[f] else (vals, rowlen[f])
    finally:
      lib.recml_parse_multi_free(handle)
    return out

  def parse_sequence(self, rows: np.ndarray, name: str, dtype: str):
    """Feature list `name` of tf.SequenceExample records: (values, values per record, steps per record);
    the values of a record's steps are concatenated in step order."""
    lib = _lib_host()
    self.validate(rows)
    kind = 0 if dtype in ("int64", "int") else 1
    np_dt = np.int64 if kind == 0 else np.float32
    offs = np.ascontiguousarray(self.offsets[rows])
    lens = np.ascontiguousarray(self.lengths[rows])
    n = len(rows)
    args = (self.data.ctypes.data_as(ctypes.c_void_p), offs.ctypes.data_as(ctypes.c_void_p),
            lens.ctypes.data_as(ctypes.c_void_p), c_ll(n), name.encode(), ctypes.c_int(kind))
    row_len, steps = np.zeros(n, dtype=np.int64), np.zeros(n, dtype=np.int64)
    lib.recml_parse_sequence_examples(*args, None, row_len.ctypes.data_as(ctypes.c_void_p),
                                      steps.ctypes.data_as(ctypes.c_void_p), None)
    starts = np.zeros(n, dtype=np.int64)
    np.cumsum(row_len[:-1], out=starts[1:])
    vals = np.empty(int(row_len.sum()), dtype=np_dt)
    lib.recml_parse_sequence_examples(*args, vals.ctypes.data_as(ctypes.c_void_p), None, None,
                                      starts.ctypes.data_as(ctypes.c_void_p))
    return vals, row_len, steps


def encode_sequence_example(context: Mapping[str, Sequence], feature_lists: Mapping[str, Sequence[Sequence]]) -> bytes:
  """Serialises a tf.train.SequenceExample: `context` like `encode_example`, `feature_lists` maps a name
  to a list of steps, each a list of ints or floats."""
  def feature(vals):
    vals = list(vals)
    if vals and isinstance(vals[0], (float, np.floating)):
      return _ld(2, _ld(1, struct.pack(f"<{len(vals)}f", *vals)))
    return _ld(3, _ld(1, b"".join(_varint(int(v)) for v in vals)))
  ctx = encode_example(context)        # Example{features=1} has the same wire shape as SequenceExample.context
  lists = b""
  for name, steps in feature_lists.items():
    fl = b"".join(_ld(1, feature(st)) for st in steps)
    lists += _ld(1, _ld(1, name.encode()) + _ld(2, fl))
  return ctx + _ld(2, lists)
