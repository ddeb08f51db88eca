"""Accuracy-style metrics reduced with `Mean`
(`recml/core/metrics/mean_metrics.py:21-112`, which defers to `keras.metrics.*`)."""
from __future__ import annotations

import torch

from recml_b200.metrics import reduction


def _t(x, like=None):
  if isinstance(x, torch.Tensor):
    return x.detach()
  return torch.as_tensor(x, device=None if like is None else like.device)


def accuracy(y_true, y_pred, weights=None, **_) -> reduction.Mean:
  """Sparse categorical accuracy: argmax(y_pred[..., C]) == y_true[...]."""
  y_pred = _t(y_pred)
  y_true = _t(y_true, y_pred)
  if y_true.ndim == y_pred.ndim and y_true.shape[-1] == 1:
    y_true = y_true.squeeze(-1)
  hit = (y_pred.argmax(dim=-1) == y_true.to(torch.int64)).to(torch.float32)
  return reduction.mean(hit, weights)


def top_k_accuracy(y_true, y_pred, weights=None, *, k: int, **_) -> reduction.Mean:
  """1 where the true class is among the k best logits.  Like Keras' `in_top_k`, the
  target counts as a hit when fewer than k classes score STRICTLY higher."""
  y_pred = _t(y_pred).to(torch.float32)
  y_true = _t(y_true, y_pred).to(torch.int64)
  if y_true.ndim == y_pred.ndim and y_true.shape[-1] == 1:
    y_true = y_true.squeeze(-1)
  target = y_pred.gather(-1, y_true.unsqueeze(-1))
  better = (y_pred > target).sum(dim=-1)
  return reduction.mean((better < k).to(torch.float32), weights)


def binary_accuracy(y_true, y_pred, weights=None, *, threshold: float = 0.5, **_) -> reduction.Mean:
  """Elementwise (y_pred > threshold) == y_true, weighted per element."""
  y_pred = _t(y_pred).to(torch.float32)
  y_true = _t(y_true, y_pred).to(torch.float32)
  hit = ((y_pred > threshold).to(torch.float32) == y_true).to(torch.float32)
  return reduction.mean(hit, weights)


def mean_squared_error(y_true, y_pred, weights=None, **_) -> reduction.Mean:
  """Keras semantics: squared error averaged over the last axis, then `Mean`."""
  y_pred = _t(y_pred).to(torch.float32)
  y_true = _t(y_true, y_pred).to(torch.float32)
  se = (y_pred - y_true) ** 2
  if se.ndim >= 1:
    se = se.mean(dim=-1)
  return reduction.mean(se, weights)
