"""Synthetic input generators for the performance configurations: Zipf ids, log-normal dense
features, Bernoulli labels, power-law sequence lengths and exponential timestamp gaps.

The reference's own generators draw uniform ids (`recml/examples/dlrm_experiment.py:204-235`,
`recml/inference/models/jax/DLRM_DCNv2/dataloader.py:38-79`); skewed ids are what makes the
embedding backward hard (a few rows receive a large share of all updates), so the benchmark
inputs here are Zipf-distributed per table.
"""
from __future__ import annotations

from typing import Iterator, Sequence

import numpy as np
import torch

from recml_b200.embedding.jagged import KeyedJagged

# Criteo-1TB table sizes and multi-hot bag sizes used by the reference's DLRM-DCNv2
# (`recml/inference/models/jax/DLRM_DCNv2/dlrm_main.py:57-65`).
CRITEO_VOCAB_SIZES = (40000000, 39060, 17295, 7424, 20265, 3, 7122, 1543, 63, 40000000, 3067956,
                      405282, 10, 2209, 11938, 155, 4, 976, 14, 40000000, 40000000, 40000000, 590152,
                      12973, 108, 36)
CRITEO_MULTI_HOT_SIZES = (3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1)


def zipf_ids(rng: np.random.Generator, vocab: int, shape, alpha: float = 1.05) -> np.ndarray:
  """Bounded Zipf(alpha) over [0, vocab) by inverting the continuous power-law CDF
  (rank r has probability ∝ r^-alpha; rank 1 ↔ id 0)."""
  u = rng.random(shape)
  if abs(alpha - 1.0) < 1e-9:
    x = np.exp(u * np.log(vocab + 1.0))
  else:
    a = 1.0 - alpha
    x = (((vocab + 1.0) ** a - 1.0) * u + 1.0) ** (1.0 / a)
  return np.clip(np.floor(x).astype(np.int64) - 1, 0, vocab - 1).astype(np.int32)


def zipf_head_shares(vocab: int, alpha: float = 1.05, rows: int = 16) -> list[float]:
  """Probabilities of ids 0 .. rows-1 (the most frequent ones) under `zipf_ids`."""
  k = np.arange(min(rows, vocab), dtype=np.float64)
  if abs(alpha - 1.0) < 1e-9:
    p = (np.log(k + 2.0) - np.log(k + 1.0)) / np.log(vocab + 1.0)
  else:
    a = 1.0 - alpha
    p = ((k + 2.0) ** a - (k + 1.0) ** a) / ((vocab + 1.0) ** a - 1.0)
  return [float(x) for x in p]


def zipf_head_share(vocab: int, alpha: float = 1.05) -> float:
  """Probability of id 0 (the most frequent one) under `zipf_ids`."""
  return zipf_head_shares(vocab, alpha, 1)[0]


def lognormal_dense(rng: np.random.Generator, batch: int, num_dense: int = 13) -> np.ndarray:
  """log(1 + LogNormal(0, 1)) per dense feature."""
  return np.log1p(rng.lognormal(0.0, 1.0, size=(batch, num_dense))).astype(np.float32)


def powerlaw_lengths(rng: np.random.Generator, n: int, lo: int = 16, hi: int = 4096, alpha: float = 1.2,
                     ) -> np.ndarray:
  """Truncated power law on [lo, hi]: p(L) ∝ L^-alpha."""
  u = rng.random(n)
  a = 1.0 - alpha
  x = ((hi ** a - lo ** a) * u + lo ** a) ** (1.0 / a)
  return np.clip(np.round(x), lo, hi).astype(np.int64)


def exponential_timestamps(rng: np.random.Generator, lengths: np.ndarray, mean_gap: float = 3600.0,
                           start: float = 1.6e9) -> np.ndarray:
  """Per-sequence increasing timestamps with Exponential(mean_gap) gaps, packed."""
  total = int(lengths.sum())
  gaps = rng.exponential(mean_gap, size=total)
  ts = np.cumsum(gaps)
  starts = np.concatenate([[0], np.cumsum(lengths)[:-1]])
  base = np.repeat(ts[starts] - gaps[starts], lengths)
  return (start + ts - base).astype(np.int64)


class DLRMBatch(dict):
  """{"dense": [B, 13] f32, "sparse": KeyedJagged, "label": [B] f32}."""

  def batch_size(self) -> int:
    return int(self["dense"].shape[0])


def make_dlrm_batch(rng: np.random.Generator, batch: int, vocab_sizes: Sequence[int],
                    bag_sizes: Sequence[int], *, num_dense: int = 13, alpha: float = 1.05,
                    pos_rate: float = 0.25, names: Sequence[str] | None = None, pin: bool = False) -> dict:
  names = list(names) if names is not None else [f"cat_{i}" for i in range(len(vocab_sizes))]
  vals = [zipf_ids(rng, v, (batch, b), alpha).reshape(-1) for v, b in zip(vocab_sizes, bag_sizes)]
  lens = np.concatenate([np.full(batch, b, dtype=np.int64) for b in bag_sizes])
  offsets = np.zeros(lens.size + 1, dtype=np.int32)
  offsets[1:] = np.cumsum(lens)
  kjt = KeyedJagged(tuple(names), torch.from_numpy(np.concatenate(vals)), torch.from_numpy(offsets), None, batch)
  out = {"dense": torch.from_numpy(lognormal_dense(rng, batch, num_dense)), "sparse": kjt,
         "label": torch.from_numpy((rng.random(batch) < pos_rate).astype(np.float32))}
  if pin and torch.cuda.is_available():
    out = {"dense": out["dense"].pin_memory(), "sparse": kjt.pin_memory(), "label": out["label"].pin_memory()}
  return out


class SyntheticDLRMDataset:
  """Cycles through `num_batches` pre-generated batches (per-rank seed) — an endless iterable."""

  def __init__(self, batch: int, vocab_sizes, bag_sizes, *, num_batches: int = 4, seed: int = 0,
               rank: int = 0, alpha: float = 1.05, pin: bool = False, steps: int | None = None,
               num_dense: int = 13):
    rng = np.random.default_rng(seed * 9973 + rank)
    self.batches = [make_dlrm_batch(rng, batch, vocab_sizes, bag_sizes, alpha=alpha, pin=pin,
                                    num_dense=num_dense) for _ in range(num_batches)]
    self.steps = steps

  def __iter__(self) -> Iterator[dict]:
    i = 0
    while self.steps is None or i < self.steps:
      yield self.batches[i % len(self.batches)]
      i += 1


def make_hstu_batch(rng: np.random.Generator, num_sequences: int, vocab: int, *, min_len: int = 16,
                    max_len: int = 4096, mean_target: int = 512, alpha_len: float = 1.2, alpha_ids: float = 1.05,
                    num_negatives: int = 512, token_capacity: int | None = None) -> dict:
    """Packed next-item batch: power-law lengths, Zipf item ids, Exponential(1 h) timestamp gaps,
    shared uniform negatives.  Lengths are rescaled so their mean is close to `mean_target` and the
    total fits `token_capacity`."""
    lens = powerlaw_lengths(rng, num_sequences, min_len, max_len, alpha_len).astype(np.float64)
    lens = np.clip(np.round(lens * mean_target / max(lens.mean(), 1.0)), min_len, max_len).astype(np.int64)
    if token_capacity is not None:
        while lens.sum() > token_capacity:
            lens[np.argmax(lens)] = max(min_len, lens.max() // 2)
    T = int(lens.sum())
    ids = zipf_ids(rng, vocab, (T + 1,), alpha_ids)
    offs = np.zeros(num_sequences + 1, dtype=np.int32)
    offs[1:] = np.cumsum(lens)
    targets = ids[1:T + 1].copy()
    weights = np.ones(T, dtype=np.float32)
    weights[offs[1:] - 1] = 0.0                      # the last position of a sequence has no next item
    return {"input_ids": torch.from_numpy(ids[:T].copy()), "target_ids": torch.from_numpy(targets),
            "negative_ids": torch.from_numpy(rng.integers(0, vocab, num_negatives).astype(np.int32)),
            "seq_offsets": torch.from_numpy(offs), "timestamps": torch.from_numpy(exponential_timestamps(rng, lens)),
            "target_weights": torch.from_numpy(weights)}
