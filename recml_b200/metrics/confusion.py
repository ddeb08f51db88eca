"""Thresholded confusion-matrix metrics: precision, recall, F-beta, AUC-PR, AUC-ROC,
precision-at-recall (`recml/core/metrics/confusion_metrics.py:24-619`).

The reference counts tp/tn/fp/fn with a vmap over thresholds — O(N·T) work.  Here the
counts come from two weighted histograms (positives, negatives) over threshold bins
and a suffix sum — O(N + T) — which is also what the fused BCE kernel emits on the
GPU (`recml_b200.ops.bce`).  A prediction p is "predicted positive at threshold t"
iff p > t (strict), so with ascending thresholds its bin is  #{t : t < p}.
"""
from __future__ import annotations

from typing import Any, Sequence

import numpy as np
import torch

from recml_b200.metrics import base

EPSILON = 1e-7


def default_thresholds(num_thresholds: int) -> np.ndarray:
  """[-eps, 1/(n-1), …, (n-2)/(n-1), 1+eps]  (`confusion_metrics.py:600-609`)."""
  inner = [(i + 1) / (num_thresholds - 1) for i in range(num_thresholds - 2)]
  return np.array([-EPSILON] + inner + [1.0 + EPSILON])


def confusion_from_histograms(pos_hist: torch.Tensor, neg_hist: torch.Tensor):
  """`hist[b]` = weight of examples with exactly b thresholds strictly below them
  (b in 0..T).  Returns tp, tn, fp, fn, each `[T]`."""
  # predicted positive at threshold k  <=>  bin > k
  pos_above = pos_hist.flip(0).cumsum(0).flip(0)  # [T+1]: Σ_{b>=k}
  neg_above = neg_hist.flip(0).cumsum(0).flip(0)
  tp, fp = pos_above[1:], neg_above[1:]
  fn, tn = pos_hist.sum() - tp, neg_hist.sum() - fp
  return tp, tn, fp, fn


def _np_div(x, y):
  x, y = np.asarray(x, dtype=np.float64), np.asarray(y, dtype=np.float64)
  with np.errstate(divide="ignore", invalid="ignore"):
    return np.where(y == 0, 0.0, x / np.where(y == 0, 1.0, y))


def _squeeze1(x):
  return x[0] if len(x) == 1 else x


def estimate_confusion_matrix(predictions, labels, weights=None,
                              thresholds: Sequence[float] = (0.0,)):
  """tp, tn, fp, fn per threshold, each of shape `[len(thresholds)]`."""
  predictions = base.as_float_tensor(predictions)
  labels_t = torch.as_tensor(np.asarray(labels) if not isinstance(labels, torch.Tensor)
                             else labels, device=predictions.device)
  if predictions.shape != labels_t.shape:
    raise ValueError("Predictions and labels must have the same shape. Got"
                     f" {tuple(predictions.shape)} and {tuple(labels_t.shape)} respectively.")
  if weights is not None:
    weights = base.as_float_tensor(weights, predictions)
    if weights.ndim != predictions.ndim:
      if weights.ndim > predictions.ndim or tuple(weights.shape) != tuple(
          predictions.shape[:weights.ndim]):
        raise ValueError("Weights are not broadcastable to predictions shape. Got the"
                         f" following shapes for predictions: {tuple(predictions.shape)}"
                         f" and weights: {tuple(weights.shape)}.")
      weights = weights.reshape(tuple(weights.shape) + (1,) * (predictions.ndim - weights.ndim))
      weights = weights.expand(predictions.shape)
    elif weights.shape != predictions.shape:
      raise ValueError("Predictions and weights must have the same shape. Got"
                       f" {tuple(predictions.shape)} and {tuple(weights.shape)} respectively.")
  th = torch.as_tensor(np.asarray(thresholds, dtype=np.float32), device=predictions.device)
  order = torch.argsort(th)
  th_sorted = th[order]
  T = th.numel()
  p = predictions.reshape(-1)
  # bin = number of thresholds strictly below p
  bins = torch.searchsorted(th_sorted, p.contiguous(), right=False)
  is_pos = labels_t.reshape(-1).to(torch.bool)
  w = torch.ones_like(p) if weights is None else weights.reshape(-1)
  pos_hist = torch.zeros(T + 1, dtype=torch.float32, device=p.device)
  neg_hist = torch.zeros(T + 1, dtype=torch.float32, device=p.device)
  pos_hist.index_add_(0, bins, w * is_pos)
  neg_hist.index_add_(0, bins, w * (~is_pos))
  tp, tn, fp, fn = confusion_from_histograms(pos_hist, neg_hist)
  inv = torch.empty_like(order)
  inv[order] = torch.arange(T, device=order.device)
  return tp[inv], tn[inv], fp[inv], fn[inv]


class ConfusionMetric(base.Metric):
  true_positives: Any
  true_negatives: Any
  false_positives: Any
  false_negatives: Any

  @classmethod
  def from_model_output(cls, y_true, y_pred, weights=None, *, threshold=0.5, **_):
    th = list(threshold) if isinstance(threshold, (Sequence, np.ndarray)) else [threshold]
    tp, tn, fp, fn = estimate_confusion_matrix(y_pred, y_true, weights, th)
    return cls(true_positives=tp, true_negatives=tn, false_positives=fp, false_negatives=fn)

  @classmethod
  def from_histograms(cls, pos_hist, neg_hist, **extra):
    """State from the two `[T+1]` histograms emitted by the fused loss kernel."""
    tp, tn, fp, fn = confusion_from_histograms(pos_hist, neg_hist)
    return cls(true_positives=tp, true_negatives=tn, false_positives=fp,
               false_negatives=fn, **extra)

  def merge(self, other):
    return self.replace(
        true_positives=self.true_positives + other.true_positives,
        true_negatives=self.true_negatives + other.true_negatives,
        false_positives=self.false_positives + other.false_positives,
        false_negatives=self.false_negatives + other.false_negatives)

  def _np(self):
    return tuple(np.asarray(base.to_numpy(x), dtype=np.float64) for x in (
        self.true_positives, self.true_negatives, self.false_positives, self.false_negatives))

  def compute(self):
    raise NotImplementedError


class Precision(ConfusionMetric):
  def compute(self):
    tp, _, fp, _ = self._np()
    return _squeeze1(_np_div(tp, tp + fp))


class Recall(ConfusionMetric):
  def compute(self):
    tp, _, _, fn = self._np()
    return _squeeze1(_np_div(tp, tp + fn))


class FBeta(ConfusionMetric):
  beta: float = 1.0

  @classmethod
  def from_model_output(cls, y_true, y_pred, weights=None, *, threshold=0.5, beta=1.0, **_):
    th = list(threshold) if isinstance(threshold, (Sequence, np.ndarray)) else [threshold]
    tp, tn, fp, fn = estimate_confusion_matrix(y_pred, y_true, weights, th)
    return cls(true_positives=tp, true_negatives=tn, false_positives=fp,
               false_negatives=fn, beta=beta)

  def compute(self):
    tp, _, fp, fn = self._np()
    p, r = _np_div(tp, tp + fp), _np_div(tp, tp + fn)
    # Same expression as the reference (`confusion_metrics.py:140-153`).
    return _squeeze1(_np_div(p * r * (self.beta + 1.0), p * self.beta + r))


class AUCPR(ConfusionMetric):
  """Area under the precision-recall curve, Davis & Goadrich interpolation."""

  @classmethod
  def from_model_output(cls, y_true, y_pred, weights=None, *, from_logits=False,
                        num_thresholds=200, **_):
    y_pred = base.as_float_tensor(y_pred)
    if from_logits:
      y_pred = torch.sigmoid(y_pred)
    tp, tn, fp, fn = estimate_confusion_matrix(
        y_pred, y_true, weights, default_thresholds(num_thresholds))
    return cls(true_positives=tp, true_negatives=tn, false_positives=fp, false_negatives=fn)

  def compute(self):
    tp, _, fp, fn = self._np()
    n = tp.shape[0]
    d_tp = tp[:n - 1] - tp[1:]
    p = tp + fp
    d_p = p[:n - 1] - p[1:]
    slope = _np_div(d_tp, np.maximum(d_p, 0))
    intercept = tp[1:] - slope * p[1:]
    both = np.logical_and(p[:n - 1] > 0, p[1:] > 0)
    ratio = np.where(both, _np_div(p[:n - 1], np.maximum(p[1:], 0)), 1.0)
    inc = _np_div(slope * (d_tp + intercept * np.log(ratio)), np.maximum(tp[1:] + fn[1:], 0))
    return float(np.sum(inc))


class _FromHistograms(base.Metric):
  """Curve metric whose state is the pair of `[T+1]` prediction histograms of the fused loss kernel (weight of
  positives / negatives with exactly b thresholds below the prediction).  Histograms add like confusion counts do,
  so steps and ranks merge by addition, and the suffix sums that turn them into tp / fp / fn / tn are taken once,
  on the host, when the value is asked for: nothing but the loss kernel runs inside the training step."""
  pos_hist: Any
  neg_hist: Any

  def merge(self, other):
    return self.replace(pos_hist=self.pos_hist + other.pos_hist, neg_hist=self.neg_hist + other.neg_hist)

  def _curve(self):
    raise NotImplementedError

  def compute(self):
    hp = torch.as_tensor(np.asarray(base.to_numpy(self.pos_hist), dtype=np.float64))
    hn = torch.as_tensor(np.asarray(base.to_numpy(self.neg_hist), dtype=np.float64))
    tp, tn, fp, fn = confusion_from_histograms(hp, hn)
    return self._curve()(true_positives=tp, true_negatives=tn, false_positives=fp, false_negatives=fn).compute()


class HistogramAUCPR(_FromHistograms):
  def _curve(self):
    return AUCPR


class HistogramAUCROC(_FromHistograms):
  def _curve(self):
    return AUCROC


class AUCROC(AUCPR):
  def compute(self):
    tp, tn, fp, fn = self._np()
    tpr, fpr = _np_div(tp, tp + fn), _np_div(fp, fp + tn)
    # thresholds ascend, so fpr descends: negate the trapezoid integral.
    return float(-np.trapezoid(tpr, fpr))


class PrecisionAtRecall(ConfusionMetric):
  recall: float = 0.1

  @classmethod
  def from_model_output(cls, y_true, y_pred, weights=None, *, num_thresholds=200,
                        recall=0.1, **_):
    tp, tn, fp, fn = estimate_confusion_matrix(
        y_pred, y_true, weights, default_thresholds(num_thresholds))
    return cls(true_positives=tp, true_negatives=tn, false_positives=fp,
               false_negatives=fn, recall=recall)

  def merge(self, other):
    if self.recall != other.recall:
      raise ValueError("Recalls must be the same to merge PrecisionAtRecall metrics.")
    return super().merge(other)

  def compute(self):
    tp, _, fp, fn = self._np()
    recalls, precisions = _np_div(tp, tp + fn), _np_div(tp, tp + fp)
    return float(precisions[int(np.argmin(np.abs(recalls - self.recall)))])


def precision(y_true, y_pred, weights=None, *, threshold=0.5, **_) -> Precision:
  return Precision.from_model_output(y_true, y_pred, weights, threshold=threshold)


def recall(y_true, y_pred, weights=None, *, threshold=0.5, **_) -> Recall:
  return Recall.from_model_output(y_true, y_pred, weights, threshold=threshold)


def fbeta_score(y_true, y_pred, weights=None, *, beta, threshold=0.5, **_) -> FBeta:
  return FBeta.from_model_output(y_true, y_pred, weights, beta=beta, threshold=threshold)


def f1_score(y_true, y_pred, weights=None, *, threshold=0.5, **_) -> FBeta:
  return fbeta_score(y_true, y_pred, weights, beta=1.0, threshold=threshold)


def aucpr(y_true, y_pred, weights=None, *, from_logits=False, num_thresholds=200, **_) -> AUCPR:
  return AUCPR.from_model_output(y_true, y_pred, weights, from_logits=from_logits,
                                 num_thresholds=num_thresholds)


def aucroc(y_true, y_pred, weights=None, *, from_logits=False, num_thresholds=200, **_) -> AUCROC:
  return AUCROC.from_model_output(y_true, y_pred, weights, from_logits=from_logits,
                                  num_thresholds=num_thresholds)


def precision_at_recall(y_true, y_pred, weights=None, *, recall=0.1, num_thresholds=200,
                        **_) -> PrecisionAtRecall:
  return PrecisionAtRecall.from_model_output(y_true, y_pred, weights, recall=recall,
                                             num_thresholds=num_thresholds)
