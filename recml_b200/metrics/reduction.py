"""Sum / Mean reductions with the reference's weight-broadcast rules
(`recml/core/metrics/reduction_metrics.py:27-227`)."""
from __future__ import annotations

import math
from typing import Any, Callable

import torch

from recml_b200.metrics import base


def align_values_and_weights(values: torch.Tensor, weights: torch.Tensor):
  """Makes `weights` elementwise-compatible with `values`.

  Same rank: each weight dim must equal the value dim or be 1.  Different rank: the
  shorter shape must be a PREFIX of the longer one and gets trailing unit dims.
  """
  vs, ws = tuple(values.shape), tuple(weights.shape)
  if vs == ws:
    return values, weights
  if len(vs) == len(ws):
    if all(v == w or w == 1 for v, w in zip(vs, ws)):
      return values, weights.expand(vs)
    raise ValueError(f"Got incompatible shapes {vs} and {ws}.")
  if len(vs) > len(ws) and vs[:len(ws)] == ws:
    return values, weights.reshape(ws + (1,) * (len(vs) - len(ws))).expand(vs)
  if len(ws) > len(vs) and ws[:len(vs)] == vs:
    return values.reshape(vs + (1,) * (len(ws) - len(vs))), weights
  raise ValueError(
      "The arrays must have the same shape or the shape of one array must be"
      f" a broadcastable to the other. Got shapes: {vs} and {ws}.")


class ReductionMetric(base.Metric):
  @classmethod
  def from_fun(cls, fun: Callable[..., Any], **bound) -> type["ReductionMetric"]:
    """A metric class computing `fun(*args, **kw)` first, then this reduction."""
    parent = cls

    class _FromFun(parent):  # pylint: disable=too-few-public-methods
      @classmethod
      def from_model_output(cls, *args, **kwargs):
        weights = kwargs.pop("weights", None)
        return parent.from_model_output(fun(*args, **bound, **kwargs), weights)

    return _FromFun


class Sum(ReductionMetric):
  total: Any

  @classmethod
  def from_model_output(cls, values, weights=None, **_) -> "Sum":
    values = base.as_float_tensor(values)
    if weights is not None:
      values, weights = align_values_and_weights(values, base.as_float_tensor(weights, values))
      return cls(total=(values * weights).sum())
    return cls(total=values.sum())

  def merge(self, other: "Sum") -> "Sum":
    return type(self)(total=self.total + other.total)

  def compute(self):
    return base.to_numpy(self.total)


class Mean(ReductionMetric):
  total: Any
  count: Any

  @classmethod
  def from_model_output(cls, values, weights=None, **_) -> "Mean":
    values = base.as_float_tensor(values)
    if weights is not None:
      values, weights = align_values_and_weights(values, base.as_float_tensor(weights, values))
      return cls(total=(values * weights).sum(), count=weights.sum())
    if values.ndim >= 1:
      n = float(math.prod(values.shape))
      return cls(total=values.sum(), count=torch.tensor(n, device=values.device))
    return cls(total=values, count=torch.ones((), device=values.device))

  def merge(self, other: "Mean") -> "Mean":
    return type(self)(total=self.total + other.total, count=self.count + other.count)

  def compute(self):
    return base.to_numpy(self.total) / base.to_numpy(self.count)


def mean(values, weights=None, **_) -> Mean:
  """total = Σ values·weights, count = Σ weights; value = total / count."""
  return Mean.from_model_output(values, weights)


def sum(values, weights=None, **_) -> Sum:  # pylint: disable=redefined-builtin
  return Sum.from_model_output(values, weights)
