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


# ---- structured masks (padding ∧ optional causality) on the tcgen05 attention kernels ----------------------
class _JaggedSoftmaxFn(torch.autograd.Function):
  """Softmax attention over packed sequences: q, k, v `[T, H, Dh]` bf16, `seq_offsets [B+1]`."""

  @staticmethod
  def forward(ctx, q, k, v, seq_offsets, max_seq_len, causal, scale, dropout_p=0.0):
    from recml_b200.ops import hstu_cuda
    from recml_b200.ops.hstu_attention import _draw_dropout
    drop = _draw_dropout(dropout_p, q.device)
    out, lse = hstu_cuda.softmax_forward(q, k, v, seq_offsets, max_seq_len, causal, scale, dropout=drop)
    ctx.save_for_backward(q, k, v, out, lse, seq_offsets)
    ctx.meta = (max_seq_len, causal, scale)
    ctx.drop = drop
    return out

  @staticmethod
  def backward(ctx, do):
    from recml_b200.ops import hstu_cuda
    q, k, v, out, lse, seq_offsets = ctx.saved_tensors
    dq, dk, dv = hstu_cuda.softmax_backward(do, out, lse, q, k, v, seq_offsets, *ctx.meta, dropout=ctx.drop)
    return dq, dk, dv, None, None, None, None, None


def jagged_softmax_attention(q, k, v, seq_offsets, max_seq_len: int, causal: bool, scale: float | None = None,
                             dropout_p: float = 0.0):
  """`dropout_p` > 0 drops attention weights inside the kernels (a counter-based hash of head, query token and
  key token seeded by one random key per call; the backward pass recomputes the same mask)."""
  scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
  from recml_b200.ops import hstu_cuda
  return _JaggedSoftmaxFn.apply(hstu_cuda.as_rows(q), hstu_cuda.as_rows(k), hstu_cuda.as_rows(v), seq_offsets, max_seq_len,
                                causal, scale, dropout_p)


def _kernel_ok(q, L: int) -> bool:
  if not q.is_cuda or q.shape[-1] not in (64, 128):
    return False
  from recml_b200.ops import hstu_cuda
  return hstu_cuda.available()


def structured_attention(q, k, v, padding_mask: torch.Tensor | None, causal: bool, dropout_p: float = 0.0,
                         training: bool = False):
  """Attention whose mask is `key is not padding` ∧ (`key <= query` when causal): q, k, v `[B, L, H, Dh]`,
  `padding_mask [B, L]` (True = real token).  On a GPU (head dim 64 / 128) the valid
  tokens are packed and run through the jagged tcgen05 kernels in softmax mode (streaming softmax, any
  length), so no `[B, H, L, L]` score tensor is ever written; rows of padded queries come back as zeros
  (the dense formulation gives them the average of the visible values; nothing downstream reads them).
  Packing happens on the device without a host synchronisation: every real token goes to its rank among
  the real tokens, padding goes to a spare row, and the kernels see `B * L` rows of capacity.
  Everywhere else this is `softmax_attention` with the merged mask."""
  B, L, H, Dh = q.shape
  drop = dropout_p if training else 0.0
  if not _kernel_ok(q, L):
    mask = merge_masks(B, L, q.device, padding_mask=padding_mask, causal=causal)
    return softmax_attention(q, k, v, mask, dropout_p, training)
  dt = q.dtype
  flat = lambda t: t.reshape(B * L, H, Dh).to(torch.bfloat16)
  if padding_mask is None:
    offs = torch.arange(B + 1, device=q.device, dtype=torch.int32) * L
    out = jagged_softmax_attention(flat(q), flat(k), flat(v), offs, L, causal, dropout_p=drop)
    return out.reshape(B, L, H, Dh).to(dt)
  T = B * L
  valid = padding_mask.bool().reshape(T)
  rank = torch.cumsum(valid, 0, dtype=torch.int32) - 1
  dest = torch.where(valid, rank, torch.full_like(rank, T)).long()       # padding lands in the spare row T
  offs = torch.zeros(B + 1, dtype=torch.int32, device=q.device)
  offs[1:] = valid.reshape(B, L).sum(1).cumsum(0)
  pack = lambda t: torch.zeros(T + 1, H, Dh, dtype=torch.bfloat16, device=q.device).index_copy(0, dest, flat(t))[:T]
  packed = jagged_softmax_attention(pack(q), pack(k), pack(v), offs, L, causal, dropout_p=drop)
  # (rows past the last real token are never written by the kernels: select, do not multiply)
  out = torch.where(valid[:, None, None], packed.index_select(0, dest.clamp(max=T - 1)), torch.zeros((), dtype=packed.dtype, device=q.device))
  return out.reshape(B, L, H, Dh).to(dt)
