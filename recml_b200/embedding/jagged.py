"""Jagged (variable-length) id features.

`KeyedJagged` packs all sparse features of a batch into two flat arrays so that one
batch needs two host→device copies regardless of the number of features:
  values  [nnz]            int32 ids, feature-major then sample-major
  offsets [F·B + 1]        int32, bag (f, b) is values[offsets[f·B+b] : offsets[f·B+b+1]]
  weights [nnz] (optional) float32 per-id gains
The reference feeds dense `[B, L]` id matrices or CSR buffers produced on the host
(`recml/layers/linen/sparsecore.py:290-354`); this container is the GPU-side equivalent.
"""
from __future__ import annotations

import dataclasses
from typing import Mapping, Sequence

import numpy as np
import torch

from recml_b200.data import iterator as iterator_lib


@dataclasses.dataclass
class KeyedJagged:
  keys: tuple[str, ...]
  values: torch.Tensor
  offsets: torch.Tensor
  weights: torch.Tensor | None = None
  _batch: int | None = None

  def __post_init__(self):
    self.keys = tuple(self.keys)
    if self._batch is None:
      self._batch = (self.offsets.numel() - 1) // max(len(self.keys), 1)

  # -- construction ----------------------------------------------------------------------
  @classmethod
  def from_dense(cls, features: Mapping[str, np.ndarray | torch.Tensor],
                 weights: Mapping[str, np.ndarray | torch.Tensor] | None = None) -> "KeyedJagged":
    """Every feature is a `[B, L_f]` (or `[B]`) id matrix: bags of fixed size L_f."""
    keys = tuple(features)
    vals, lens, ws = [], [], []
    batch = None
    for k in keys:
      x = torch.as_tensor(np.asarray(features[k]) if not isinstance(features[k], torch.Tensor)
                          else features[k])
      if x.ndim == 1:
        x = x[:, None]
      batch = x.shape[0] if batch is None else batch
      vals.append(x.reshape(-1).to(torch.int32))
      lens.append(torch.full((x.shape[0],), x.shape[1], dtype=torch.int32))
      if weights is not None:
        w = weights.get(k)
        ws.append(torch.ones(x.numel()) if w is None else
                  torch.as_tensor(np.asarray(w), dtype=torch.float32).reshape(-1))
    lengths = torch.cat(lens) if lens else torch.zeros(0, dtype=torch.int32)
    offsets = torch.zeros(lengths.numel() + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(lengths, 0)
    return cls(keys, torch.cat(vals) if vals else torch.zeros(0, dtype=torch.int32), offsets,
               torch.cat(ws).to(torch.float32) if weights is not None else None, batch or 0)

  @classmethod
  def from_lists(cls, features: Mapping[str, Sequence[Sequence[int]]],
                 weights: Mapping[str, Sequence[Sequence[float]]] | None = None) -> "KeyedJagged":
    keys = tuple(features)
    vals, lens, ws = [], [], []
    for k in keys:
      for b, bag in enumerate(features[k]):
        vals.extend(int(v) for v in bag)
        lens.append(len(bag))
        if weights is not None:
          ws.extend((weights[k][b] if k in weights else [1.0] * len(bag)))
    offsets = np.zeros(len(lens) + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(lens)
    batch = len(next(iter(features.values()))) if keys else 0
    return cls(keys, torch.tensor(vals, dtype=torch.int32), torch.from_numpy(offsets),
               torch.tensor(ws, dtype=torch.float32) if weights is not None else None, batch)

  # -- protocol used by partitioners / trainers ----------------------------------------------
  def batch_size(self) -> int:
    return int(self._batch)

  def num_features(self) -> int:
    return len(self.keys)

  def spec(self):
    return {"keys": self.keys, "values": iterator_lib.ArraySpec((None,), self.values.dtype),
            "offsets": iterator_lib.ArraySpec(tuple(self.offsets.shape), self.offsets.dtype)}

  def to_device(self, device, stager=None) -> "KeyedJagged":
    def put(t):
      if t is None:
        return None
      if device.type == "cuda" and not t.is_cuda:
        if stager is not None:
          return stager.put(t, device)
        return t.pin_memory().to(device, non_blocking=True)
      return t.to(device)
    return KeyedJagged(self.keys, put(self.values), put(self.offsets), put(self.weights), self._batch)

  def pin_memory(self) -> "KeyedJagged":
    return KeyedJagged(self.keys, self.values.pin_memory(), self.offsets.pin_memory(),
                       None if self.weights is None else self.weights.pin_memory(), self._batch)

  def slice_batch(self, lo: int, hi: int) -> "KeyedJagged":
    B, F = self._batch, len(self.keys)
    off = self.offsets.to(torch.int64)
    vals, ws, lens = [], [], []
    for f in range(F):
      a, b = int(off[f * B + lo]), int(off[f * B + hi])
      vals.append(self.values[a:b])
      if self.weights is not None:
        ws.append(self.weights[a:b])
      lens.append((off[f * B + lo + 1:f * B + hi + 1] - off[f * B + lo:f * B + hi]).to(torch.int32))
    lengths = torch.cat(lens)
    offsets = torch.zeros(lengths.numel() + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(lengths, 0)
    return KeyedJagged(self.keys, torch.cat(vals), offsets,
                       torch.cat(ws) if self.weights is not None else None, hi - lo)

  def feature(self, key: str) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor | None]:
    """(values, offsets rebased to 0, weights) of one feature."""
    f, B = self.keys.index(key), self._batch
    off = self.offsets[f * B:(f + 1) * B + 1].to(torch.int64)
    a, b = int(off[0]), int(off[-1])
    return (self.values[a:b], off - off[0],
            None if self.weights is None else self.weights[a:b])

  def to_lists(self) -> dict[str, list[list[int]]]:
    out = {}
    for k in self.keys:
      v, o, _ = self.feature(k)
      out[k] = [v[int(o[i]):int(o[i + 1])].tolist() for i in range(self._batch)]
    return out
