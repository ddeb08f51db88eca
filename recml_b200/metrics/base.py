"""Metric state objects.

A metric is a small frozen record of tensors ("state") produced on the device inside
the training / evaluation step by `from_model_output`, pulled to the host with
`localize()` (device tensors become numpy arrays), folded across steps with `merge`
and turned into a number with `compute`, which uses numpy only.  This is the contract
of the reference's `Metric` (`recml/core/metrics/base_metrics.py:35-104`) restated for
torch tensors; `reduce_across_ranks` is added because each process here owns one GPU.
"""
from __future__ import annotations

import abc
import dataclasses
import math
from typing import Any, Mapping, Sequence

import numpy as np
import torch

Scalar = float | Sequence[float] | Mapping[str, float] | np.ndarray | torch.Tensor


def as_float_tensor(x: Any, like: torch.Tensor | None = None) -> torch.Tensor:
  if isinstance(x, torch.Tensor):
    return x.detach().to(torch.float32)
  device = like.device if isinstance(like, torch.Tensor) else None
  return torch.as_tensor(np.asarray(x), dtype=torch.float32, device=device)


def to_numpy(x: Any) -> Any:
  if isinstance(x, torch.Tensor):
    return x.detach().to("cpu").numpy()
  return x


class Metric(abc.ABC):
  """Base class; subclasses are frozen dataclasses of tensors / python scalars."""

  def __init_subclass__(cls, **kwargs):
    super().__init_subclass__(**kwargs)
    dataclasses.dataclass(frozen=True, eq=False)(cls)

  @classmethod
  def from_model_output(cls, *args, **kwargs) -> "Metric":
    raise NotImplementedError

  @abc.abstractmethod
  def merge(self, other: "Metric") -> "Metric":
    """Combines two states of the same type (host side; `+` on arrays only)."""

  @abc.abstractmethod
  def compute(self) -> Scalar:
    """Final value from the (localized) state; numpy only."""

  def replace(self, **updates) -> "Metric":
    return dataclasses.replace(self, **updates)

  def localize(self) -> "Metric":
    """Copy of the state with every tensor moved to host numpy."""
    return self.replace(**{f.name: to_numpy(getattr(self, f.name))
                           for f in dataclasses.fields(self)})

  def start_localize(self, stream: "torch.cuda.Stream | None" = None) -> "Metric":
    """Non-blocking device→pinned-host copies; call `.localize()` on the result later."""
    out = {}
    for f in dataclasses.fields(self):
      v = getattr(self, f.name)
      if isinstance(v, torch.Tensor) and v.is_cuda:
        host = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
        with torch.cuda.stream(stream or torch.cuda.current_stream()):
          host.copy_(v, non_blocking=True)
        v = host
      out[f.name] = v
    return self.replace(**out)

  def reduce_across_ranks(self, group=None) -> "Metric":
    """Sums every tensor field over the process group (for sum-type states)."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
      return self
    out = {}
    for f in dataclasses.fields(self):
      v = getattr(self, f.name)
      if isinstance(v, (torch.Tensor, np.ndarray)):
        t = torch.as_tensor(v).clone()
        if dist.get_backend(group) == "nccl" and not t.is_cuda:
          t = t.cuda()
        dist.all_reduce(t, group=group)
        v = t
      out[f.name] = v
    return self.replace(**out)


class ScalarMetric(Metric):
  """Reports a value as-is; on merge the most recent observation wins
  (`recml/core/metrics/base_metrics.py:107-154`)."""

  value: Any

  @classmethod
  def from_model_output(cls, value) -> "ScalarMetric":
    shape = getattr(value, "shape", ())
    if math.prod(shape) != 1:
      raise ValueError(f"Scalar metric values must be scalars. Got shape: {tuple(shape)}")
    return cls(value=as_float_tensor(value).reshape(()))

  def merge(self, other: "ScalarMetric") -> "ScalarMetric":
    return other

  def compute(self) -> Scalar:
    return to_numpy(self.value)

  def reduce_across_ranks(self, group=None) -> "ScalarMetric":
    return self


def scalar(value) -> ScalarMetric:
  """Per-step scalar (learning rate, batch loss): last value wins when merged."""
  return ScalarMetric.from_model_output(value)
