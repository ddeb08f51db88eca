"""Fused binary cross-entropy with logits: loss, gradient and metric statistics in one pass.

Reference semantics: `mean(max(x,0) − x·y + log1p(exp(−|x|)))` (`recml/examples/
dlrm_experiment.py:274-277`) and the task metrics built from the same logits — label /
prediction means, accuracy at logit 0, AUC-PR / AUC-ROC from 200-threshold confusion counts
(`dlrm_experiment.py:284-292`, `recml/core/metrics/confusion_metrics.py:567-609`).  The kernel
emits two weighted histograms over the threshold bins from which all confusion counts follow
by a suffix sum, so the O(N·T) vmap of the reference becomes O(N + T).
"""
from __future__ import annotations

import ctypes
import dataclasses

import torch

from recml_b200.metrics import confusion
from recml_b200.ops import _lib


@dataclasses.dataclass
class BCEResult:
  loss_sum: torch.Tensor       # Σ loss·w
  weight_sum: torch.Tensor     # Σ w
  label_sum: torch.Tensor
  pred_sum: torch.Tensor
  correct_sum: torch.Tensor
  dlogits: torch.Tensor | None
  hist_pos: torch.Tensor | None
  hist_neg: torch.Tensor | None

  @property
  def loss(self) -> torch.Tensor:
    return self.loss_sum / self.weight_sum


def _auc_bins(p: torch.Tensor, T: int) -> torch.Tensor:
  th = torch.as_tensor(confusion.default_thresholds(T), dtype=torch.float32, device=p.device)
  return torch.searchsorted(th, p.contiguous(), right=False)


def bce_with_logits(logits: torch.Tensor, labels: torch.Tensor, weights: torch.Tensor | None = None, *,
                    grad_scale: float | None = None, num_thresholds: int = 200,
                    grad_dtype: torch.dtype = torch.float32) -> BCEResult:
  """`grad_scale` None → no gradient; else dlogits = (σ(x) − y)·w·grad_scale (pass 1/global_batch
  for a mean loss).  `num_thresholds` 0 disables the histograms."""
  n, T = logits.numel(), num_thresholds
  logits = logits.reshape(-1)
  labels = labels.reshape(-1).to(torch.float32)
  if not logits.is_cuda:
    x = logits.to(torch.float32)
    w = torch.ones_like(x) if weights is None else weights.reshape(-1).to(torch.float32)
    p = torch.sigmoid(x)
    loss = torch.clamp(x, min=0) - x * labels + torch.log1p(torch.exp(-x.abs()))
    hp = hn = None
    if T:
      bins = _auc_bins(p, T)
      hp = torch.zeros(T + 1).index_add_(0, bins, w * (labels > 0.5))
      hn = torch.zeros(T + 1).index_add_(0, bins, w * (labels <= 0.5))
    d = None if grad_scale is None else ((p - labels) * w * grad_scale).to(grad_dtype)
    return BCEResult((loss * w).sum(), w.sum(), (labels * w).sum(), (p * w).sum(),
                     (((x > 0) == (labels > 0.5)) * w).sum(), d, hp, hn)
  dev = logits.device
  stats = torch.zeros(8, dtype=torch.float32, device=dev)
  hist = torch.zeros(2, T + 1, dtype=torch.float32, device=dev) if T else None
  d32 = d16 = None
  if grad_scale is not None:
    if grad_dtype == torch.bfloat16:
      d16 = torch.empty(n, dtype=torch.bfloat16, device=dev)
    else:
      d32 = torch.empty(n, dtype=torch.float32, device=dev)
  logits = logits.contiguous()
  rc = _lib.cuda().recml_bce_logits(
      _lib.ptr(logits), ctypes.c_int(int(logits.dtype == torch.bfloat16)), _lib.ptr(labels.contiguous()),
      _lib.ptr(None if weights is None else weights.reshape(-1).to(torch.float32).contiguous()),
      ctypes.c_longlong(n), ctypes.c_float(grad_scale or 0.0), _lib.ptr(d32), _lib.ptr(d16), _lib.ptr(stats),
      _lib.ptr(None if hist is None else hist[0]), _lib.ptr(None if hist is None else hist[1]),
      ctypes.c_int(T), _lib.stream())
  _lib.check_rc(rc, "recml_bce_logits")
  return BCEResult(stats[0], stats[1], stats[2], stats[3], stats[4], d32 if d32 is not None else d16,
                   None if hist is None else hist[0], None if hist is None else hist[1])


class _BCEFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, logits, labels, weights, scale):
    r = bce_with_logits(logits.detach(), labels, weights, grad_scale=scale, num_thresholds=0,
                        grad_dtype=torch.float32)
    ctx.save_for_backward(r.dlogits)
    ctx.shape, ctx.dtype = logits.shape, logits.dtype
    return r.loss_sum * scale

  @staticmethod
  def backward(ctx, g):
    (d,) = ctx.saved_tensors
    return (d * g).to(ctx.dtype).view(ctx.shape), None, None, None


def bce_loss(logits, labels, weights=None, *, scale: float | None = None) -> torch.Tensor:
  """Differentiable scalar Σ loss·w·scale (default scale = 1/numel → mean)."""
  return _BCEFn.apply(logits, labels, weights, scale if scale is not None else 1.0 / logits.numel())
