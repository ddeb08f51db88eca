"""Array storage for checkpoints: one zarr-v2 array directory per tree leaf.

This is the layout Orbax's PyTree handler writes when OCDBT is off (a checkpoint is
recognised as OCDBT by the presence of `manifest.ocdbt`): `<item>/<dotted.leaf.key>/
.zarray` plus C-order chunk files named by dot-joined chunk indices.  Chunks are written
uncompressed ("compressor": null) or zstd-compressed when libzstd can be loaded;
both are valid zarr v2 and readable by TensorStore.  Sharded leaves are ONE global
array whose chunk grid equals the shard grid, so every rank writes only its own chunk
files and any world size can read any region back.

Bulk byte movement goes through the native writer in `csrc/ckpt/` when it is built.
"""
from __future__ import annotations

import ctypes
import ctypes.util
import json
import os
from typing import Sequence

import numpy as np
import torch

_ZARR_DTYPES = {
    np.dtype("float32"): "<f4", np.dtype("float64"): "<f8", np.dtype("float16"): "<f2",
    np.dtype("int64"): "<i8", np.dtype("int32"): "<i4", np.dtype("int16"): "<i2",
    np.dtype("int8"): "|i1", np.dtype("uint8"): "|u1", np.dtype("bool"): "|b1",
    np.dtype("uint16"): "<u2", np.dtype("uint32"): "<u4", np.dtype("uint64"): "<u8",
}
_FROM_ZARR = {v: k for k, v in _ZARR_DTYPES.items()}
BFLOAT16 = "bfloat16"  # TensorStore's zarr driver spells bf16 this way


def _zstd():
  for name in ("libzstd.so.1", ctypes.util.find_library("zstd")):
    if not name:
      continue
    try:
      lib = ctypes.CDLL(name)
    except OSError:
      continue
    lib.ZSTD_compressBound.restype = ctypes.c_size_t
    lib.ZSTD_compressBound.argtypes = [ctypes.c_size_t]
    lib.ZSTD_compress.restype = ctypes.c_size_t
    lib.ZSTD_compress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                  ctypes.c_size_t, ctypes.c_int]
    lib.ZSTD_decompress.restype = ctypes.c_size_t
    lib.ZSTD_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p,
                                    ctypes.c_size_t]
    lib.ZSTD_isError.restype = ctypes.c_uint
    lib.ZSTD_isError.argtypes = [ctypes.c_size_t]
    if hasattr(lib, "ZSTD_compress2"):          # the context API (1.4+): frames with a content checksum
      lib.ZSTD_createCCtx.restype = ctypes.c_void_p
      lib.ZSTD_freeCCtx.argtypes = [ctypes.c_void_p]
      lib.ZSTD_CCtx_setParameter.restype = ctypes.c_size_t
      lib.ZSTD_CCtx_setParameter.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
      lib.ZSTD_compress2.restype = ctypes.c_size_t
      lib.ZSTD_compress2.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
    return lib
  return None


_ZSTD = _zstd()


def zstd_available() -> bool:
  return _ZSTD is not None


_ZSTD_C_LEVEL, _ZSTD_C_CHECKSUM, _ZSTD_C_WORKERS = 100, 201, 400   # compressionLevel, checksumFlag, nbWorkers
_ZSTD_MT_BYTES = 8 << 20          # inputs from this size on are compressed by several threads


def zstd_compress(raw, level: int = 1) -> bytes:
  """One standard zstd frame from `bytes` or a contiguous numpy array (no copy of the input).  With the context
  API the frame carries a content checksum (XXH64, four bytes at its end), which every zstd reader verifies
  while decompressing: a flipped bit in a stored chunk is an error at restore instead of a wrong weight.
  Large inputs use the library's worker threads when it was built with them (the frame stays standard)."""
  if isinstance(raw, np.ndarray):
    raw = np.ascontiguousarray(raw)
    src, n_src = ctypes.c_void_p(raw.ctypes.data), raw.nbytes
  else:
    src, n_src = raw, len(raw)
  bound = _ZSTD.ZSTD_compressBound(n_src)
  dst = ctypes.create_string_buffer(bound)
  if hasattr(_ZSTD, "ZSTD_compress2"):
    cctx = _ZSTD.ZSTD_createCCtx()
    try:
      _ZSTD.ZSTD_CCtx_setParameter(cctx, _ZSTD_C_LEVEL, level)
      _ZSTD.ZSTD_CCtx_setParameter(cctx, _ZSTD_C_CHECKSUM, 1)
      if n_src >= _ZSTD_MT_BYTES:      # an error (a single-threaded build of the library) leaves one thread
        _ZSTD.ZSTD_CCtx_setParameter(cctx, _ZSTD_C_WORKERS, min(8, os.cpu_count() or 1))
      n = _ZSTD.ZSTD_compress2(cctx, dst, bound, src, n_src)
    finally:
      _ZSTD.ZSTD_freeCCtx(cctx)
  else:
    n = _ZSTD.ZSTD_compress(dst, bound, src, n_src, level)
  if _ZSTD.ZSTD_isError(n):
    raise IOError("zstd compression failed")
  return ctypes.string_at(dst, n)


def zstd_decompress(blob: bytes, raw_size: int) -> bytes:
  out = np.empty(raw_size, dtype=np.uint8)
  zstd_decompress_into(blob, out)
  return out.tobytes()


def zstd_decompress_into(blob: bytes, out: np.ndarray) -> None:
  """Decompresses one frame straight into `out` (contiguous, exactly the decompressed size in bytes)."""
  n = _ZSTD.ZSTD_decompress(ctypes.c_void_p(out.ctypes.data), out.nbytes, blob, len(blob))
  if _ZSTD.ZSTD_isError(n) or n != out.nbytes:
    raise IOError("zstd decompression failed (truncated or corrupt chunk)")


def to_host_numpy(t, copy: bool = False) -> tuple[np.ndarray, str]:
  """Returns (array viewable as bytes, zarr dtype string).  A tensor that already lives in host memory is
  returned as a VIEW of that memory unless `copy` is set: a caller that writes it later, while training goes on
  (an asynchronous save), must ask for the copy."""
  if isinstance(t, torch.Tensor):
    t = t.detach()
    host = t.cpu().contiguous()
    if copy and host.data_ptr() == t.data_ptr():
      host = host.clone()
    if t.dtype == torch.bfloat16:
      return host.view(torch.int16).numpy(), BFLOAT16
    arr = host.numpy()
  else:
    arr = np.array(t, copy=True) if copy else np.ascontiguousarray(np.asarray(t))
    arr = np.ascontiguousarray(arr)
  if arr.dtype not in _ZARR_DTYPES:
    raise TypeError(f"Unsupported checkpoint dtype {arr.dtype}")
  return arr, _ZARR_DTYPES[arr.dtype]


def write_zarray(path: str, shape: Sequence[int], chunks: Sequence[int], dtype: str,
                 compressor: str | None) -> None:
  os.makedirs(path, exist_ok=True)
  meta = {
      "chunks": [int(c) for c in chunks] if len(shape) else [],
      "compressor": ({"id": "zstd", "level": 1} if compressor == "zstd" else None),
      "dimension_separator": ".", "dtype": dtype, "fill_value": None, "filters": None,
      "order": "C", "shape": [int(s) for s in shape], "zarr_format": 2,
  }
  with open(os.path.join(path, ".zarray"), "w") as f:
    json.dump(meta, f)


def chunk_name(index: Sequence[int]) -> str:
  return ".".join(str(int(i)) for i in index) if len(index) else "0"


def write_chunk(path: str, index: Sequence[int], arr: np.ndarray, compressor: str | None) -> None:
  raw = arr.tobytes(order="C")
  if compressor == "zstd":
    raw = zstd_compress(raw)
  tmp = os.path.join(path, "." + chunk_name(index) + ".partial")
  with open(tmp, "wb") as f:
    f.write(raw)
  os.replace(tmp, os.path.join(path, chunk_name(index)))


def write_array(path: str, value, compressor: str | None = None) -> None:
  """Whole array as a single chunk."""
  arr, dtype = to_host_numpy(value)
  write_zarray(path, arr.shape, arr.shape, dtype, compressor)
  write_chunk(path, [0] * arr.ndim, arr, compressor)


def _is_ocdbt(path: str) -> bool:
  return path.startswith("ocdbt:")


def _ocdbt_get(path: str, name: str) -> bytes:
  """Value of `<array key>/<name>` for an array that lives in an OCDBT store (`ckpt/ocdbt.py`)."""
  from recml_b200.ckpt import ocdbt
  store_dir, key = ocdbt.split_path(path)
  return ocdbt.open_store(store_dir).get(f"{key}/{name}" if key else name)


def read_meta(path: str) -> dict:
  if _is_ocdbt(path):
    return json.loads(_ocdbt_get(path, ".zarray"))
  with open(os.path.join(path, ".zarray")) as f:
    return json.load(f)


def _np_dtype(zdtype: str) -> np.dtype:
  return np.dtype("int16") if zdtype == BFLOAT16 else _FROM_ZARR[zdtype]


def read_region(path: str, start: Sequence[int] | None = None,
                stop: Sequence[int] | None = None) -> torch.Tensor:
  """Reads `[start, stop)` of the array (default: all of it) from whatever chunk grid
  it was written with.  Missing chunk files raise FileNotFoundError (half-written
  checkpoints are detected this way by continuous evaluation)."""
  meta = read_meta(path)
  shape, chunks = meta["shape"], meta["chunks"]
  dt = _np_dtype(meta["dtype"])
  comp = meta.get("compressor")
  nd = len(shape)
  start = [0] * nd if start is None else list(start)
  stop = list(shape) if stop is None else list(stop)
  out = np.empty([b - a for a, b in zip(start, stop)], dtype=dt)
  if out.size == 0:                      # an empty leaf (or an empty request) has no chunk to read
    t = torch.from_numpy(out)
    return t.view(torch.bfloat16) if meta["dtype"] == BFLOAT16 else t
  if nd >= 1 and comp is None and _read_rows_native(path, shape, chunks, dt, start, stop, out):
    t = torch.from_numpy(out)
    return t.view(torch.bfloat16) if meta["dtype"] == BFLOAT16 else t
  if nd >= 1 and comp is None and _is_ocdbt(path) and (
      _read_whole_chunk_ocdbt(path, shape, chunks, start, stop, out) or
      _read_rows_ocdbt(path, shape, chunks, dt, start, stop, out)):
    t = torch.from_numpy(out)
    return t.view(torch.bfloat16) if meta["dtype"] == BFLOAT16 else t
  if nd == 0:
    out = np.array(_read_chunk(path, [], [], dt, comp, []).reshape(()))      # a writable 0-d copy
  else:
    lo = [a // c for a, c in zip(start, chunks)]
    hi = [(b - 1) // c for b, c in zip(stop, chunks)]
    for idx in np.ndindex(*[h - l + 1 for l, h in zip(lo, hi)]):
      cidx = [l + i for l, i in zip(lo, idx)]
      c0 = [ci * c for ci, c in zip(cidx, chunks)]
      data = _read_chunk(path, cidx, chunks, dt, comp, shape)
      # zarr stores edge chunks at full chunk shape; clip to the array and to the request
      src = tuple(slice(max(a, o) - o, min(b, o + c, s) - o)
                  for a, b, o, c, s in zip(start, stop, c0, chunks, shape))
      dst = tuple(slice(max(a, o) - a, min(b, o + c, s) - a)
                  for a, b, o, c, s in zip(start, stop, c0, chunks, shape))
      out[dst] = data[src]
  t = torch.from_numpy(out)            # `out` is contiguous and owned here (ascontiguousarray would turn 0-d into 1-d)
  return t.view(torch.bfloat16) if meta["dtype"] == BFLOAT16 else t


_SEGMENT_BYTES = 16 << 20


def _checksums_enabled() -> bool:
  return os.environ.get("RECML_CKPT_CHECKSUMS", "1") != "0"


def _checksum_path(chunk_path: str) -> str:
  d, name = os.path.split(chunk_path)
  return os.path.join(d, "." + name + ".crc32c")


def _write_checksums(chunk_path: str, crcs: list[int]) -> None:
  tmp = _checksum_path(chunk_path) + ".partial"
  with open(tmp, "w") as f:
    json.dump({"segment_bytes": _SEGMENT_BYTES, "crc32c": crcs}, f)
  os.replace(tmp, _checksum_path(chunk_path))


def _stored_checksums(chunk_path: str) -> list[int] | None:
  """The segment checksums written beside a raw chunk, or None (another writer, an older checkpoint, checks
  switched off with RECML_CKPT_CHECKSUMS=0)."""
  if not _checksums_enabled():
    return None
  try:
    with open(_checksum_path(chunk_path)) as f:
      doc = json.load(f)
  except (OSError, ValueError):
    return None
  if doc.get("segment_bytes") != _SEGMENT_BYTES:
    return None
  return [int(c) for c in doc.get("crc32c", [])]


def _verify_segments(chunk_path: str, lib, base_ptr: int, nbytes: int, want: list[int]) -> None:
  k = (nbytes + _SEGMENT_BYTES - 1) // _SEGMENT_BYTES
  if k != len(want):
    raise IOError(f"{chunk_path}: {len(want)} stored checksums for {k} segments")
  bufs = (ctypes.c_void_p * k)(*[base_ptr + i * _SEGMENT_BYTES for i in range(k)])
  sizes = (ctypes.c_longlong * k)(*[min(_SEGMENT_BYTES, nbytes - i * _SEGMENT_BYTES) for i in range(k)])
  got = (ctypes.c_uint32 * k)()
  lib.recml_crc32c_many(ctypes.c_int(k), bufs, sizes, got)
  for i in range(k):
    if int(got[i]) != want[i]:
      raise IOError(f"{chunk_path}: checksum mismatch in bytes [{i * _SEGMENT_BYTES}, "
                    f"{i * _SEGMENT_BYTES + int(sizes[i])}) — the chunk is damaged")


def _write_raw_native(lib, items) -> None:
  """Uncompressed chunks straight from the arrays' memory (no intermediate copy): each chunk goes to a
  `.partial` file created at its final size, written in 16 MB segments by all host threads, then renamed."""
  arrays = [np.ascontiguousarray(arr) for _, _, arr in items]       # kept alive until the write returns
  finals = [os.path.join(path, chunk_name(index)) for path, index, _ in items]
  segs = []
  for arr, final in zip(arrays, finals):
    tmp = final + ".partial"
    with open(tmp, "wb") as f:
      f.truncate(arr.nbytes)
    base = arr.ctypes.data
    for off in range(0, arr.nbytes, _SEGMENT_BYTES):
      segs.append((tmp.encode(), off, base + off, min(_SEGMENT_BYTES, arr.nbytes - off)))
  n = len(segs)
  if n:
    paths = (ctypes.c_char_p * n)(*[s[0] for s in segs])
    offs = (ctypes.c_longlong * n)(*[s[1] for s in segs])
    bufs = (ctypes.c_void_p * n)(*[s[2] for s in segs])
    sizes = (ctypes.c_longlong * n)(*[s[3] for s in segs])
    rc = lib.recml_write_ranges(ctypes.c_int(n), paths, offs, bufs, sizes)
    if rc != 0:
      raise IOError(f"native chunk write failed for {segs[-rc - 1][0].decode()}")
    if _checksums_enabled() and hasattr(lib, "recml_crc32c_many"):
      # CRC-32C of every 16 MB segment, kept in a dot-file beside the chunk (array-store readers ignore it):
      # raw chunks carry no checksum of their own, so a flipped bit would otherwise restore as a wrong weight
      crcs = (ctypes.c_uint32 * n)()
      lib.recml_crc32c_many(ctypes.c_int(n), bufs, sizes, crcs)
      at = 0
      for arr, final in zip(arrays, finals):
        k = (arr.nbytes + _SEGMENT_BYTES - 1) // _SEGMENT_BYTES
        _write_checksums(final, [int(c) for c in crcs[at:at + k]])
        at += k
  for final in finals:
    os.rename(final + ".partial", final)


def _read_whole_chunk_ocdbt(path, shape, chunks, start, stop, out: np.ndarray) -> bool:
  """A raw chunk of an OCDBT store that is exactly the requested region (a leaf or a shard stored as one chunk
  and read back whole): its value is read straight into `out` by the store's parallel reader.  False: the
  caller takes the general path."""
  cidx = [a // c if c else 0 for a, c in zip(start, chunks)]
  for d, ci in enumerate(cidx):
    c0 = ci * chunks[d]
    if start[d] != c0 or stop[d] != min(c0 + chunks[d], shape[d]) or (stop[d] - start[d] != chunks[d] and d > 0):
      return False
  from recml_b200.ckpt import ocdbt
  store_dir, leaf = ocdbt.split_path(path)
  store = ocdbt.open_store(store_dir)
  key = f"{leaf}/{chunk_name(cidx)}"
  try:
    if store.value_size(key) != out.nbytes:
      return False                       # a clipped or padded chunk: the general path sorts it out
  except FileNotFoundError:
    raise FileNotFoundError(os.path.join(path, chunk_name(cidx))) from None
  store.read_into(key, out)
  return True


def _read_rows_ocdbt(path, shape, chunks, dt, start, stop, out: np.ndarray) -> bool:
  """Raw arrays of an OCDBT store chunked along the first dimension only, whole rows requested (a rank taking
  its rows out of a table that another world size saved): only the bytes of the requested rows are read from
  each chunk's value, straight into `out`.  False: the caller takes the general path."""
  nd = len(shape)
  if any(chunks[d] != shape[d] or start[d] != 0 or stop[d] != shape[d] for d in range(1, nd)) or out.size == 0:
    return False
  from recml_b200.ckpt import ocdbt
  store_dir, leaf = ocdbt.split_path(path)
  store = ocdbt.open_store(store_dir)
  row_bytes = int(np.prod(shape[1:], dtype=np.int64)) * dt.itemsize if nd > 1 else dt.itemsize
  a, b, c = start[0], stop[0], chunks[0]
  flat = out.reshape(-1).view(np.uint8)
  plan = []
  for ci in range(a // c, (b - 1) // c + 1):
    key = f"{leaf}/{chunk_name([ci] + [0] * (nd - 1))}"
    lo, hi = max(a, ci * c), min(b, (ci + 1) * c, shape[0])
    f_off, d_off, size = (lo - ci * c) * row_bytes, (lo - a) * row_bytes, (hi - lo) * row_bytes
    try:
      if store.value_size(key) < f_off + size:
        return False                     # a foreign chunk layout: the general path sorts it out
    except FileNotFoundError:
      raise FileNotFoundError(os.path.join(path, chunk_name([ci] + [0] * (nd - 1)))) from None
    plan.append((key, f_off, d_off, size))
  for key, f_off, d_off, size in plan:
    store.read_range_into(key, f_off, flat[d_off:d_off + size])
  return True


def _read_rows_native(path, shape, chunks, dt, start, stop, out: np.ndarray) -> bool:
  """Uncompressed arrays chunked along the first dimension only, whole rows requested: every chunk maps
  to one contiguous piece of `out`, so the native reader fills `out` directly, many threads at once and
  in segments of 16 MB (a table shard is one large chunk).  False: the caller takes the general path."""
  nd = len(shape)
  if _is_ocdbt(path):
    return False
  if any(chunks[d] != shape[d] or start[d] != 0 or stop[d] != shape[d] for d in range(1, nd)) or out.size == 0:
    return False
  try:
    from recml_b200.ops import _lib
    lib = _lib.host()
  except Exception:  # pylint: disable=broad-except
    return False
  if lib is None or not hasattr(lib, "recml_read_ranges"):
    return False
  row_bytes = int(np.prod(shape[1:], dtype=np.int64)) * dt.itemsize if nd > 1 else dt.itemsize
  a, b, c = start[0], stop[0], chunks[0]
  items = []
  for ci in range(a // c, (b - 1) // c + 1):
    fpath = os.path.join(path, chunk_name([ci] + [0] * (nd - 1)))
    if not os.path.exists(fpath):
      raise FileNotFoundError(fpath)
    lo, hi = max(a, ci * c), min(b, (ci + 1) * c, shape[0])
    f_off, d_off, size = (lo - ci * c) * row_bytes, (lo - a) * row_bytes, (hi - lo) * row_bytes
    if os.path.getsize(fpath) < f_off + size:
      return False                      # clipped or foreign chunk layout
    for seg in range(0, size, _SEGMENT_BYTES):
      items.append((fpath.encode(), f_off + seg, d_off + seg, min(_SEGMENT_BYTES, size - seg)))
  n = len(items)
  base = out.ctypes.data
  whole = []          # (path, offset in out, bytes) of every chunk file read from its first to its last byte
  for ci in range(a // c, (b - 1) // c + 1):
    fpath = os.path.join(path, chunk_name([ci] + [0] * (nd - 1)))
    lo, hi = max(a, ci * c), min(b, (ci + 1) * c, shape[0])
    if lo == ci * c and (hi - lo) * row_bytes == os.path.getsize(fpath):
      whole.append((fpath, (lo - a) * row_bytes, (hi - lo) * row_bytes))
  paths = (ctypes.c_char_p * n)(*[it[0] for it in items])
  offs = (ctypes.c_longlong * n)(*[it[1] for it in items])
  bufs = (ctypes.c_void_p * n)(*[base + it[2] for it in items])
  sizes = (ctypes.c_longlong * n)(*[it[3] for it in items])
  rc = lib.recml_read_ranges(ctypes.c_int(n), paths, offs, bufs, sizes, ctypes.c_int(0))
  if rc != 0:
    raise IOError(f"native chunk read failed for {items[-rc - 1][0].decode()}")
  if hasattr(lib, "recml_crc32c_many"):
    for fpath, d_off, nbytes in whole:        # a range inside a chunk cannot be checked against segment sums
      want = _stored_checksums(fpath)
      if want is not None:
        _verify_segments(fpath, lib, base + d_off, nbytes, want)
  return True


def _verify_blob(chunk_path: str, blob: bytes, want: list[int]) -> None:
  try:
    from recml_b200.ops import _lib
    lib = _lib.host()
  except Exception:  # pylint: disable=broad-except
    return
  if lib is None or not hasattr(lib, "recml_crc32c_many"):
    return
  buf = np.frombuffer(blob, dtype=np.uint8)
  _verify_segments(chunk_path, lib, buf.ctypes.data, buf.size, want)


def _read_chunk(path, cidx, chunks, dt, comp, shape) -> np.ndarray:
  """One chunk at full chunk shape.  A stored chunk holds either the full chunk or, for the last chunk along the
  first dimension, exactly the rows that exist (a writer that clips its edge chunk); any other size is a
  damaged file and raises instead of restoring zeros."""
  name = chunk_name(cidx)
  if _is_ocdbt(path):
    blob = _ocdbt_get(path, name)
  else:
    with open(os.path.join(path, name), "rb") as f:
      blob = f.read()
  n = int(np.prod(chunks)) if len(chunks) else 1
  raw = comp is None
  if not raw:
    if comp.get("id") != "zstd" or not zstd_available():
      raise IOError(f"Unsupported chunk compressor {comp}")
    full = np.empty(n, dtype=dt)               # zstd chunks are always stored at full chunk shape
    zstd_decompress_into(blob, full.view(np.uint8).reshape(-1) if n else full.view(np.uint8))
    return full.reshape(chunks) if len(chunks) else full[:1]
  clipped = -1
  if len(chunks):
    rows = min(int(chunks[0]), int(shape[0]) - int(cidx[0]) * int(chunks[0]))
    clipped = rows * (n // int(chunks[0])) * dt.itemsize if chunks[0] else 0
  if len(blob) not in (n * dt.itemsize, clipped):
    raise IOError(f"{os.path.join(path, name)}: chunk holds {len(blob)} bytes, expected {n * dt.itemsize}"
                  + (f" (or {clipped} for the clipped last chunk)" if 0 <= clipped < n * dt.itemsize else ""))
  if raw and not _is_ocdbt(path):            # compressed chunks carry their own content checksum
    want = _stored_checksums(os.path.join(path, name))
    if want is not None:
      _verify_blob(os.path.join(path, name), blob, want)
  if len(blob) == n * dt.itemsize:
    return np.frombuffer(blob, dtype=dt, count=n).reshape(chunks) if len(chunks) else \
        np.frombuffer(blob, dtype=dt, count=1)
  arr = np.zeros(n, dtype=dt)
  part = np.frombuffer(blob, dtype=dt)
  arr[:part.size] = part
  return arr.reshape(chunks)


def write_chunks_parallel(items, compressor: str | None = None) -> None:
  """`items`: list of (array dir, chunk index, numpy array).  Chunks are written concurrently by the
  native chunk writer (`csrc/ckpt/chunk_io.cpp`: temp name + rename per chunk); falls back to the
  serial Python writer when the native library is unavailable."""
  if not items:
    return
  try:
    from recml_b200.ops import _lib
    lib = _lib.host()
  except Exception:  # pylint: disable=broad-except
    lib = None
  if lib is None:
    for path, index, arr in items:
      write_chunk(path, index, arr, compressor)
    return
  if compressor is None and hasattr(lib, "recml_write_ranges"):
    _write_raw_native(lib, items)
    return
  blobs = []
  for path, index, arr in items:
    raw = zstd_compress(np.ascontiguousarray(arr)) if compressor == "zstd" else arr.tobytes(order="C")
    blobs.append((os.path.join(path, chunk_name(index)).encode(), raw))
  n = len(blobs)
  paths = (ctypes.c_char_p * n)(*[b[0] for b in blobs])
  bufs = (ctypes.c_char_p * n)(*[b[1] for b in blobs])
  sizes = (ctypes.c_longlong * n)(*[len(b[1]) for b in blobs])
  rc = lib.recml_write_chunks(ctypes.c_int(n), paths, ctypes.cast(bufs, ctypes.POINTER(ctypes.c_void_p)), sizes, None,
                              ctypes.c_int(0))
  if rc != 0:
    raise IOError(f"native chunk write failed for {blobs[-rc - 1][0].decode()}")
