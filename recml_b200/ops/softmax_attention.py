"""Softmax multi-head attention for the SASRec / BERT4Rec blocks (sequence length ≤ a few
hundred): scaled dot product with padding ∧ (causal | explicit) masks.  The math is the one the
reference gets from keras_hub's `TransformerDecoder` / `TransformerEncoder`
(`recml/layers/keras/sasrec.py:89-101`, `bert4rec.py:106-118`)."""
from __future__ import annotations

import math

import torch


def merge_masks(batch: int, length: int, device, *, padding_mask=None, attention_mask=None,
                causal: bool = False) -> torch.Tensor | None:
  """Boolean `[B, L, L]` (True = attend) from a `[B, L]` key padding mask, an explicit
  `[B, L, L]` mask and causality."""
  m = None
  if padding_mask is not None:
    m = padding_mask.bool()[:, None, :].expand(batch, length, length)
  if attention_mask is not None:
    a = attention_mask.bool()
    m = a if m is None else (m & a)
  if causal:
    c = torch.tril(torch.ones(length, length, dtype=torch.bool, device=device))[None]
    m = c.expand(batch, length, length) if m is None else (m & c)
  return m


def softmax_attention(q, k, v, mask: torch.Tensor | None, dropout_p: float = 0.0, training: bool = False):
  """q, k, v `[B, L, H, Dh]`; mask `[B, L, L]` boolean.  fp32 softmax."""
  s = torch.einsum("bthd,bshd->bhts", q.float(), k.float()) / math.sqrt(q.shape[-1])
  if mask is not None:
    s = s.masked_fill(~mask[:, None], -1e9)
  p = torch.softmax(s, dim=-1)
  if training and dropout_p > 0:
    p = torch.nn.functional.dropout(p, dropout_p)
  return torch.einsum("bhts,bshd->bthd", p, v.float()).to(q.dtype)
