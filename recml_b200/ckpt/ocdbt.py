"""OCDBT key-value stores (`csrc/ckpt/ocdbt.cpp`): the default on-disk form of the reference's checkpoints
(`manifest.ocdbt`, `d/<data files>`, `ocdbt.process_<n>/` per writing process; saved through
`ocp.CheckpointManager`, `recml/core/training/jax_trainer.py:475-484`).  Inside the store the arrays are
ordinary zarr v2: key `<leaf>/.zarray` holds the metadata and `<leaf>/<i>.<j>` the chunks.

The codec follows the public description of the format and round-trips with itself (zstd-compressed
multi-level trees, several process directories); it has not been compared with a file written by the
reference's own libraries, which are not installable here.
"""
from __future__ import annotations

import ctypes
import os

from recml_b200.ops import _lib

PREFIX = "ocdbt:"


def is_store(directory: str) -> bool:
  return os.path.exists(os.path.join(directory, "manifest.ocdbt")) or os.path.isdir(
      os.path.join(directory, "ocdbt.process_0"))


def leaf_path(store_dir: str, key: str) -> str:
  """The pseudo-path `zarr_io` understands for array `key` inside the store at `store_dir`."""
  return f"{PREFIX}{store_dir}#{key}"


def split_path(path: str) -> tuple[str, str]:
  store_dir, key = path[len(PREFIX):].split("#", 1)
  return store_dir, key


def _host():
  lib = _lib.host()
  if not getattr(lib, "_ocdbt_ready", False):
    lib.recml_ocdbt_open.restype = ctypes.c_void_p
    lib.recml_ocdbt_open.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int]
    lib.recml_ocdbt_close.argtypes = [ctypes.c_void_p]
    lib.recml_ocdbt_num_keys.restype = ctypes.c_longlong
    lib.recml_ocdbt_num_keys.argtypes = [ctypes.c_void_p]
    lib.recml_ocdbt_key.restype = ctypes.c_char_p
    lib.recml_ocdbt_key.argtypes = [ctypes.c_void_p, ctypes.c_longlong]
    lib.recml_ocdbt_value_size.restype = ctypes.c_longlong
    lib.recml_ocdbt_value_size.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
    lib.recml_ocdbt_read.restype = ctypes.c_longlong
    lib.recml_ocdbt_read.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong]
    lib.recml_ocdbt_read_range.restype = ctypes.c_longlong
    lib.recml_ocdbt_read_range.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_longlong, ctypes.c_void_p,
                                           ctypes.c_longlong]
    lib.recml_ocdbt_writer_new.restype = ctypes.c_void_p
    lib.recml_ocdbt_writer_new.argtypes = [ctypes.c_char_p, ctypes.c_longlong]
    lib.recml_ocdbt_writer_add.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong]
    lib.recml_ocdbt_writer_add_ref.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong]
    lib.recml_ocdbt_writer_commit.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    lib.recml_ocdbt_writer_abort.argtypes = [ctypes.c_void_p]
    lib._ocdbt_ready = True
  return lib


class Store:
  """Read access to every key of a store directory (its own manifest plus the per-process stores beside it)."""

  def __init__(self, directory: str):
    self._lib = _host()
    err = ctypes.create_string_buffer(512)
    self._h = self._lib.recml_ocdbt_open(directory.encode(), err, 512)
    if not self._h:
      raise IOError(f"cannot open OCDBT store {directory}: {err.value.decode(errors='replace')}")
    self.directory = directory

  def keys(self) -> list[str]:
    n = self._lib.recml_ocdbt_num_keys(self._h)
    return [self._lib.recml_ocdbt_key(self._h, i).decode() for i in range(n)]

  def __contains__(self, key: str) -> bool:
    return self._lib.recml_ocdbt_value_size(self._h, key.encode()) >= 0

  def get(self, key: str) -> bytes:
    import numpy as np
    n = self.value_size(key)
    buf = np.empty(max(n, 1), dtype=np.uint8)          # no zero fill, one copy on the way out
    got = self._lib.recml_ocdbt_read(self._h, key.encode(), buf.ctypes.data, n)
    if got != n:
      raise IOError(f"{self.directory}: reading {key!r} failed with code {got}")
    return buf[:n].tobytes()

  def value_size(self, key: str) -> int:
    n = self._lib.recml_ocdbt_value_size(self._h, key.encode())
    if n < 0:
      raise FileNotFoundError(f"{self.directory}: no key {key!r}")
    return int(n)

  def read_into(self, key: str, out) -> None:
    """The value of `key` straight into `out`, a contiguous writable numpy array of exactly its size in bytes:
    no intermediate copy, read in 16 MB pieces by all host threads."""
    n = self.value_size(key)
    if not out.flags["C_CONTIGUOUS"] or not out.flags["WRITEABLE"] or out.nbytes != n:
      raise ValueError(f"{key!r} holds {n} bytes, the buffer {out.nbytes}")
    got = self._lib.recml_ocdbt_read(self._h, key.encode(), out.ctypes.data, n)
    if got != n:
      raise IOError(f"{self.directory}: reading {key!r} failed with code {got}")

  def read_range_into(self, key: str, value_offset: int, out) -> None:
    """Bytes [value_offset, value_offset + out.nbytes) of the value of `key` into `out` (contiguous, writable):
    a row range of a large chunk without reading the rest of it."""
    if not out.flags["C_CONTIGUOUS"] or not out.flags["WRITEABLE"]:
      raise ValueError("the destination must be a contiguous writable array")
    got = self._lib.recml_ocdbt_read_range(self._h, key.encode(), int(value_offset), out.ctypes.data, out.nbytes)
    if got == -1:
      raise FileNotFoundError(f"{self.directory}: no key {key!r}")
    if got != out.nbytes:
      raise IOError(f"{self.directory}: reading {out.nbytes} bytes at {value_offset} of {key!r} failed with code {got}")

  def close(self) -> None:
    if self._h:
      self._lib.recml_ocdbt_close(self._h)
      self._h = None

  def __del__(self):
    try:
      self.close()
    except Exception:  # pylint: disable=broad-except
      pass


_open: dict[str, Store] = {}


def open_store(directory: str) -> Store:
  """A cached reader (a checkpoint's leaves are all read from the same store)."""
  key = os.path.abspath(directory)
  st = _open.get(key)
  stamp = os.path.getmtime(os.path.join(directory, "manifest.ocdbt")) if os.path.exists(
      os.path.join(directory, "manifest.ocdbt")) else None
  if st is None or getattr(st, "_stamp", None) != stamp:
    st = Store(directory)
    st._stamp = stamp
    _open[key] = st
    while len(_open) > 8:
      _open.pop(next(iter(_open)))
  return st


class Writer:
  """Collects key → bytes pairs and writes them as one store (data file + B+tree + manifest) on commit."""

  def __init__(self, directory: str, max_inline_value_bytes: int = 100):
    self._lib = _host()
    os.makedirs(directory, exist_ok=True)
    self._h = self._lib.recml_ocdbt_writer_new(directory.encode(), max_inline_value_bytes)
    self.directory = directory
    self._keep: list = []       # arrays added by reference

  def add(self, key: str, data: bytes | memoryview) -> None:
    data = bytes(data) if not isinstance(data, bytes) else data
    self._lib.recml_ocdbt_writer_add(self._h, key.encode(), data, len(data))

  def add_array(self, key: str, arr) -> None:
    """The bytes of a numpy array as the value, without a copy: the array is kept alive until the commit, which
    writes it from its own memory."""
    import numpy as np
    arr = np.ascontiguousarray(arr)
    self._keep.append(arr)
    self._lib.recml_ocdbt_writer_add_ref(self._h, key.encode(), arr.ctypes.data, arr.nbytes)

  def commit(self, compress_nodes: bool = True, node_fanout: int = 64) -> None:
    h, self._h = self._h, None
    rc = self._lib.recml_ocdbt_writer_commit(h, int(compress_nodes), node_fanout)
    self._keep = []
    if rc == -2:
      raise ValueError(f"OCDBT store {self.directory}: a key was added twice")
    if rc != 0:
      raise IOError(f"writing OCDBT store {self.directory} failed with code {rc}")

  def __del__(self):
    if getattr(self, "_h", None):
      self._lib.recml_ocdbt_writer_abort(self._h)
