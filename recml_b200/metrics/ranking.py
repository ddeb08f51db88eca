"""Ranking metrics for retrieval heads: Recall@K / HR@K, NDCG@K, MRR.

The reference advertises these (`README.md:38`) but ships only top-k accuracy
(`recml/core/metrics/mean_metrics.py:43-65`; HR@10/50/200 in
`recml/examples/train_hstu_keras.py:141-145`).  All of them are functions of the
1-based rank of the positive item:  rank = 1 + #{items scoring strictly higher}.
With a sharded vocabulary each rank counts "strictly higher" on its shard and the
counts are summed, so the full logits never exist (`recml_b200.ops.vocab_logits`).
"""
from __future__ import annotations

import math

import torch

from recml_b200.metrics import reduction


def rank_of_target(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
  """1-based rank of `targets[...]` within `logits[..., V]` (ties rank optimistically)."""
  logits = logits.detach().to(torch.float32)
  t = logits.gather(-1, targets.to(torch.int64).unsqueeze(-1))
  return 1 + (logits > t).sum(dim=-1)


def recall_at_k_from_rank(rank, k: int, weights=None) -> reduction.Mean:
  return reduction.mean((rank <= k).to(torch.float32), weights)


def ndcg_at_k_from_rank(rank, k: int, weights=None) -> reduction.Mean:
  """One relevant item: DCG = 1/log2(1+rank) if rank ≤ k, ideal DCG = 1."""
  gain = torch.where(rank <= k, 1.0 / torch.log2(1.0 + rank.to(torch.float32)),
                     torch.zeros((), device=rank.device))
  return reduction.mean(gain, weights)


def mrr_from_rank(rank, weights=None, k: int | None = None) -> reduction.Mean:
  rr = 1.0 / rank.to(torch.float32)
  if k is not None:
    rr = torch.where(rank <= k, rr, torch.zeros((), device=rank.device))
  return reduction.mean(rr, weights)


def recall_at_k(y_true, y_pred, weights=None, *, k: int, **_) -> reduction.Mean:
  return recall_at_k_from_rank(rank_of_target(torch.as_tensor(y_pred), torch.as_tensor(y_true)), k, weights)


hit_rate_at_k = recall_at_k


def ndcg_at_k(y_true, y_pred, weights=None, *, k: int, **_) -> reduction.Mean:
  return ndcg_at_k_from_rank(rank_of_target(torch.as_tensor(y_pred), torch.as_tensor(y_true)), k, weights)


def mrr(y_true, y_pred, weights=None, *, k: int | None = None, **_) -> reduction.Mean:
  return mrr_from_rank(rank_of_target(torch.as_tensor(y_pred), torch.as_tensor(y_true)), weights, k)


def ideal_dcg(num_relevant: int, k: int) -> float:
  return sum(1.0 / math.log2(2 + i) for i in range(min(num_relevant, k)))
