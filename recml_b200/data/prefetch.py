"""Host→device prefetching on a copy stream.

`DevicePrefetcher(iterator, partitioner, depth)` keeps `depth` batches in flight: the pinned-memory
H2D copies of batch i+1 … i+depth are issued on a dedicated stream while the training stream is
still computing step i, and `next()` makes the consuming stream wait only for the copy of the
batch it hands out.  It is the device-side half of the reference's threaded input producer
(`recml/inference/models/jax/DLRM_DCNv2/dlrm_main.py:174-291` keeps a queue of device-ready
batches); on CPU it degenerates to `partitioner.shard_inputs(next(iterator))`.
"""
from __future__ import annotations

import collections
from typing import Any, Iterator

import torch


def _tensors(tree, out):
  if isinstance(tree, torch.Tensor):
    out.append(tree)
  elif isinstance(tree, dict):
    for v in tree.values():
      _tensors(v, out)
  elif isinstance(tree, (list, tuple)):
    for v in tree:
      _tensors(v, out)
  elif hasattr(tree, "values") and hasattr(tree, "offsets"):      # KeyedJagged
    for t in (tree.values, tree.offsets, tree.weights):
      if t is not None:
        out.append(t)
  return out


class DevicePrefetcher:
  def __init__(self, iterator: Iterator[Any], partitioner, depth: int = 1):
    self._it = iter(iterator)
    self._part = partitioner
    self._depth = max(0, int(depth))
    device = getattr(partitioner, "device", None)
    self._cuda = device is not None and device.type == "cuda" and self._depth > 0
    self._stream = torch.cuda.Stream(device=device) if self._cuda else None
    self._device = device
    self._queue: collections.deque = collections.deque()
    self._done = False

  def _issue(self) -> None:
    try:
      host = next(self._it)
    except StopIteration:
      self._done = True
      return
    with torch.cuda.stream(self._stream):
      dev = self._part.shard_inputs(host)
      ev = torch.cuda.Event()
      ev.record(self._stream)
    self._queue.append((host, dev, ev))

  def __iter__(self):
    return self

  def __next__(self):
    batch, _ = self.next_with_host()
    return batch

  def next_with_host(self):
    """(device batch, the host batch it came from)."""
    if not self._cuda:
      host = next(self._it)
      return self._part.shard_inputs(host), host
    while not self._done and len(self._queue) < self._depth + 1:
      self._issue()
    if not self._queue:
      raise StopIteration
    host, dev, ev = self._queue.popleft()
    cur = torch.cuda.current_stream(self._device)
    cur.wait_event(ev)
    for t in _tensors(dev, []):           # allocated on the copy stream, consumed on this one
      if t.is_cuda:
        t.record_stream(cur)
    if not self._done and len(self._queue) < self._depth:
      self._issue()                        # keep the pipe full before the caller starts the step
    return dev, host
