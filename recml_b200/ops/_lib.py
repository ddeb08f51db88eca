"""ctypes bindings to the in-tree native libraries.

`cuda()` returns `librecml_cuda.so`; it raises if the library is missing or stale and
cannot be rebuilt, so a GPU run never silently falls back to library kernels.
"""
from __future__ import annotations

import ctypes
import functools
import os
from typing import Any

import torch

from recml_b200 import _build


class NativeError(RuntimeError):
  pass


# Number of this library's kernels launched so far (benchmarks reset and read it).  Each launcher
# call counts the kernels it launches (the radix sort: four per pass, counted by its caller).
LAUNCHES = {"count": 0}
_KERNELS_PER_CALL = {"recml_emb_bwd_update": 2, "recml_allreduce_bucket": 3, "recml_radix_sort_scratch_words": 0,
                     "recml_radix_sort_passes": 0, "recml_id_unique_scratch_words": 0, "recml_id_unique_sorted": 3,
                     "recml_emb_bucketize_struct_size": 0,
                     "recml_emb_struct_sizes": 0, "recml_optim_struct_sizes": 0, "recml_ar_struct_sizes": 0,
                     "recml_ssd_struct_size": 0, "recml_ssd_ckpt_interval": 0, "recml_conv1d_silu_bwd": 2,
                     "recml_hstu_struct_size": 0, "recml_vocab_rank_struct_size": 0}


class _CountingLib:
  def __init__(self, lib: ctypes.CDLL):
    self._lib = lib
    self._fns: dict[str, Any] = {}

  def __getattr__(self, name: str):
    fn = self._fns.get(name)
    if fn is None:
      raw = getattr(self._lib, name)
      n = _KERNELS_PER_CALL.get(name, 1)
      if name in ("recml_radix_sort_scratch_words", "recml_id_unique_scratch_words"):
        raw.restype = ctypes.c_longlong

      def fn(*args, _raw=raw, _n=n):
        LAUNCHES["count"] += _n
        return _raw(*args)
      self._fns[name] = fn
    return fn


@functools.lru_cache(maxsize=None)
def cuda() -> "_CountingLib":
  libs = _build.build()
  if "cuda" not in libs:
    raise NativeError("librecml_cuda.so could not be built (no CUDA sources / nvcc).")
  return _CountingLib(ctypes.CDLL(libs["cuda"]))


@functools.lru_cache(maxsize=None)
def host() -> ctypes.CDLL:
  libs = _build.build()
  if "host" not in libs:
    raise NativeError("librecml_host.so could not be built.")
  return ctypes.CDLL(libs["host"])


def ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
  return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream() -> ctypes.c_void_p:
  return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


_status: dict[int, torch.Tensor] = {}
_status_host: dict[int, torch.Tensor] = {}


def status_buffer(device: torch.device | None = None) -> torch.Tensor:
  """Per-device int32[4] word that kernels write an error code into (0 = ok)."""
  idx = torch.cuda.current_device() if device is None or device.index is None else device.index
  if idx not in _status:
    _status[idx] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", idx))
  return _status[idx]


STATUS_NAMES = {1: "mbarrier wait timed out", 2: "peer flag wait timed out", 3: "bad argument",
                4: "buffer capacity exceeded", 5: "input id outside its table (detail = the id)"}


class DeviceStatusError(RuntimeError):
  """A kernel reported a bounded-wait timeout or capacity error."""


class PeerTimeoutError(DeviceStatusError):
  pass


def check_status(device: torch.device | None = None, sync: bool = True) -> None:
  """Reads the status word (synchronising) and raises if a kernel reported an error."""
  buf = status_buffer(device)
  vals = buf.cpu().tolist() if sync else buf.tolist()
  if vals[0] != 0:
    buf.zero_()
    cls = PeerTimeoutError if vals[0] == 2 else DeviceStatusError
    raise cls(f"device status {vals[0]} ({STATUS_NAMES.get(vals[0], '?')}), detail {vals[1]}")


class _StatusPoller:
  """Looks at the status word without stalling the host: every call issues an asynchronous copy of
  the word into pinned memory and examines the copy issued by the previous call once its event has
  completed, so an error reported by a kernel surfaces one or two steps later instead of at the next
  synchronisation point."""

  def __init__(self, device: torch.device):
    self.device = device
    self.pinned = torch.zeros(2, 4, dtype=torch.int32).pin_memory()
    self.events: list[Any] = [None, None]
    self.turn = 0

  def poll(self) -> None:
    buf = status_buffer(self.device)
    prev = self.turn ^ 1
    ev = self.events[prev]
    if ev is not None and ev.query():
      vals = self.pinned[prev].tolist()
      self.events[prev] = None
      if vals[0] != 0:
        buf.zero_()
        cls = PeerTimeoutError if vals[0] == 2 else DeviceStatusError
        raise cls(f"device status {vals[0]} ({STATUS_NAMES.get(vals[0], '?')}), detail {vals[1]}")
    cur = self.turn
    if self.events[cur] is None:
      self.pinned[cur].copy_(buf, non_blocking=True)
      ev = torch.cuda.Event()
      ev.record(torch.cuda.current_stream(self.device))
      self.events[cur] = ev
      self.turn ^= 1


_pollers: dict[int, _StatusPoller] = {}


def poll_status(device: torch.device | None = None) -> None:
  """Non-blocking status check for hot loops (see `_StatusPoller`); `check_status` is the blocking one."""
  idx = torch.cuda.current_device() if device is None or device.index is None else device.index
  if idx not in _status:
    return          # no kernel of this library has run on the device yet
  if idx not in _pollers:
    _pollers[idx] = _StatusPoller(torch.device("cuda", idx))
  _pollers[idx].poll()


# ---- checked build (RECML_DEBUG=1): canary words around buffers that kernels write --------------------------
DEBUG = _build.DEBUG
_CANARY = 0x5AC0FFEE
_GUARD = 64           # int32 words before and after the payload
_guarded: list[tuple[torch.Tensor, int, str]] = []


def debug_empty(shape, dtype: torch.dtype, device, what: str = "buffer") -> torch.Tensor:
  """`torch.empty` in the optimised build.  In the checked build the tensor sits between two guard zones
  filled with a known word; `debug_check()` verifies them after the kernels that wrote the tensor have
  run, so a kernel that writes outside its output (wrong pitch, tile overhang, bad offset) is caught where
  it happens instead of corrupting a neighbour."""
  if not DEBUG:
    return torch.empty(shape, dtype=dtype, device=device)
  n = 1
  for s_ in shape:
    n *= int(s_)
  nbytes = n * torch.empty((), dtype=dtype).element_size()
  words = (nbytes + 3) // 4
  raw = torch.full((2 * _GUARD + words,), _CANARY, dtype=torch.int32, device=device)
  _guarded.append((raw, words, what))
  payload = raw[_GUARD:_GUARD + words].view(torch.uint8)[:nbytes].view(dtype)
  return payload.view(*shape)


def debug_check() -> None:
  """Verifies (and forgets) every guard zone handed out since the last call; synchronises."""
  if not DEBUG or not _guarded:
    return
  torch.cuda.synchronize()
  bad = []
  for raw, words, what in _guarded:
    head, tail = raw[:_GUARD], raw[_GUARD + words:]
    if not (bool((head == _CANARY).all()) and bool((tail == _CANARY).all())):
      bad.append(what)
  _guarded.clear()
  if bad:
    raise DeviceStatusError(f"guard words overwritten around: {', '.join(bad)}")


def check_rc(rc: int, what: str) -> None:
  if rc != 0:
    raise NativeError(f"{what} failed with code {rc}")
