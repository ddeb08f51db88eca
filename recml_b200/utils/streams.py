"""Named side streams for work that overlaps the main stream inside one training step.

The step's critical path (embedding forward → dense forward → data-gradient chain) stays on the
current stream.  Work that only has to be finished by the optimizer step is forked onto side
streams: the radix sort of the embedding occurrences ("emb_sort", under the dense forward), the
embedding backward ("emb_bwd") and the weight-gradient GEMMs ("wgrad"), which run beside each other
once the data-gradient chain is done.  `fork(name)` makes the side stream wait for everything issued
so far on the current stream and remembers that it must be joined; `join(...)` makes the current
stream wait for the named side streams (all forked ones by default).  Every forked stream is joined
before the step ends, which is also what CUDA-graph capture requires.
"""
from __future__ import annotations

import contextlib

import torch

_streams: dict[tuple[int, str], "torch.cuda.Stream"] = {}
_forked: dict[int, list[str]] = {}


def _dev_index(device=None) -> int:
  if device is None:
    return torch.cuda.current_device()
  device = torch.device(device)
  return torch.cuda.current_device() if device.index is None else device.index


def side(name: str, device=None, priority: int = 0) -> "torch.cuda.Stream":
  """The side stream called `name` on `device` (created on first use)."""
  key = (_dev_index(device), name)
  s = _streams.get(key)
  if s is None:
    s = torch.cuda.Stream(device=key[0], priority=priority)
    _streams[key] = s
  return s


def fork(name: str, device=None, priority: int = 0) -> "torch.cuda.Stream":
  """Side stream `name`, ordered after everything issued so far on the current stream."""
  idx = _dev_index(device)
  s = side(name, idx, priority)
  s.wait_stream(torch.cuda.current_stream(idx))
  names = _forked.setdefault(idx, [])
  if name not in names:
    names.append(name)
  return s


def chain(name: str, after: str, device=None) -> None:
  """Orders side stream `name` after what has been issued on side stream `after` (if it exists)."""
  idx = _dev_index(device)
  a = _streams.get((idx, after))
  if a is not None:
    side(name, idx).wait_stream(a)


def join(*names: str, device=None) -> None:
  """Makes the current stream wait for the named forked side streams (all of them when none is named)."""
  if not torch.cuda.is_available():
    return
  idx = _dev_index(device)
  pending = _forked.get(idx)
  if not pending:
    return
  cur = torch.cuda.current_stream(idx)
  for name in list(pending):
    if names and name not in names:
      continue
    cur.wait_stream(_streams[(idx, name)])
    pending.remove(name)


def keep_alive_on(stream: "torch.cuda.Stream", *tensors) -> None:
  """Tells the caching allocator that `tensors` (allocated on another stream) are read on `stream`."""
  for t in tensors:
    if t is not None and t.is_cuda:
      t.record_stream(stream)


@contextlib.contextmanager
def on(stream: "torch.cuda.Stream"):
  with torch.cuda.stream(stream):
    yield stream
