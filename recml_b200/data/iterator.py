"""Dataset iterator protocol (`recml/core/data/iterator.py:27-130`).

An `Iterator` yields batches (pytrees of numpy arrays / tensors), can describe one
element without consuming it (`element_spec`), can be rewound (`reset`) and can
save / restore its position for resumable training.
"""
from __future__ import annotations

import abc
import dataclasses
import pickle
from typing import Any, Callable, Iterable

import numpy as np
import torch


@dataclasses.dataclass(frozen=True)
class ArraySpec:
  shape: tuple[int | None, ...]
  dtype: Any


def _spec_of(x: Any) -> Any:
  if isinstance(x, dict):
    return {k: _spec_of(v) for k, v in x.items()}
  if isinstance(x, (list, tuple)):
    return type(x)(_spec_of(v) for v in x)
  if hasattr(x, "spec"):
    return x.spec()
  if isinstance(x, (np.ndarray, torch.Tensor)):
    return ArraySpec(tuple(x.shape), x.dtype)
  return ArraySpec((), type(x))


class Iterator(abc.ABC):
  """Resumable batch iterator."""

  def __iter__(self):
    return self

  @abc.abstractmethod
  def __next__(self) -> Any: ...

  @property
  @abc.abstractmethod
  def element_spec(self) -> Any: ...

  @abc.abstractmethod
  def reset(self) -> None: ...

  def save(self, filename: str) -> None:
    with open(filename, "wb") as f:
      pickle.dump(self.get_state(), f)

  def restore(self, filename: str) -> None:
    with open(filename, "rb") as f:
      self.set_state(pickle.load(f))

  def get_state(self) -> Any:
    return None

  def set_state(self, state: Any) -> None:
    del state


def _freeze(x: Any) -> Any:
  if isinstance(x, np.ndarray):
    x.setflags(write=False)
  elif isinstance(x, dict):
    for v in x.values():
      _freeze(v)
  elif isinstance(x, (list, tuple)):
    for v in x:
      _freeze(v)
  return x


class IterableIterator(Iterator):
  """Wraps any re-iterable dataset.  `postprocessor` runs on every batch on the host
  (this is where the sharded-embedding id preprocessor is attached, like the
  reference's `TFDatasetIterator(dataset, postprocessor=SparsecorePreprocessor)`).
  numpy outputs are made read-only so a step cannot corrupt a cached batch."""

  def __init__(self, dataset: Iterable, postprocessor: Callable[[Any], Any] | None = None):
    self._dataset = dataset
    self._post = postprocessor
    self._it = None
    self._position = 0
    self._peeked: list[Any] = []
    self._spec = None

  def _ensure(self):
    if self._it is None:
      self._it = iter(self._dataset)

  def _produce(self) -> Any:
    self._ensure()
    batch = next(self._it)
    if self._post is not None:
      batch = self._post(batch)
    return _freeze(batch)

  def __next__(self) -> Any:
    batch = self._peeked.pop(0) if self._peeked else self._produce()
    self._position += 1
    return batch

  @property
  def element_spec(self) -> Any:
    if self._spec is None:
      if not self._peeked:
        self._peeked.append(self._produce())
      self._spec = _spec_of(self._peeked[0])
    return self._spec

  def reset(self) -> None:
    self._it = None
    self._peeked.clear()
    self._position = 0

  def get_state(self) -> Any:
    inner = getattr(self._dataset, "get_state", lambda: None)()
    return {"position": self._position, "dataset": inner}

  def set_state(self, state: Any) -> None:
    self.reset()
    if state.get("dataset") is not None and hasattr(self._dataset, "set_state"):
      self._dataset.set_state(state["dataset"])
      self._position = state["position"]
      return
    for _ in range(state["position"]):  # generic datasets: fast-forward
      next(self)


# Name kept for users of the reference API.
TFDatasetIterator = IterableIterator
