"""Transformer blocks shared by SASRec (pre-LN decoder, causal) and BERT4Rec (post-LN encoder):
multi-head softmax attention with biases on Q, K, V, O and a two-layer feed-forward network,
three dropouts per block (attention weights, attention output, FFN output) — the structure of the
keras_hub blocks the reference instantiates (`recml/layers/keras/sasrec.py:89-101`,
`bert4rec.py:106-118`; parameter counts pinned by `sasrec_test.py:36-50`)."""
from __future__ import annotations

from typing import Callable

import torch
from torch import nn

from recml_b200.layers import utils
from recml_b200.ops import dense as dense_ops
from recml_b200.ops import norm as norm_ops
from recml_b200.ops import softmax_attention as sm_ops


def _glorot_(w):
  nn.init.xavier_uniform_(w)


class MultiHeadAttention(nn.Module):
  def __init__(self, model_dim: int, num_heads: int, dropout: float = 0.0, init: Callable = _glorot_):
    super().__init__()
    assert model_dim % num_heads == 0
    self.num_heads, self.head_dim, self.dropout_p = num_heads, model_dim // num_heads, dropout
    self.qkv = nn.Parameter(torch.empty(3 * model_dim, model_dim))   # rows: q | k | v
    for i in range(3):
      init(self.qkv.data[i * model_dim:(i + 1) * model_dim])
    self.qkv_bias = nn.Parameter(torch.zeros(3 * model_dim))
    self.out = nn.Parameter(torch.empty(model_dim, model_dim))
    init(self.out)
    self.out_bias = nn.Parameter(torch.zeros(model_dim))

  def forward(self, x: torch.Tensor, mask: torch.Tensor | None, *, padding_mask: torch.Tensor | None = None,
              causal: bool = False, structured: bool = False) -> torch.Tensor:
    """`structured` says that `mask` is exactly padding ∧ causality (no explicit attention mask), which
    lets the op use the packed-sequence kernels instead of a dense `[B, L, L]` mask."""
    B, L, D = x.shape
    qkv = dense_ops.linear(x, self.qkv, self.qkv_bias).reshape(B, L, 3, self.num_heads, self.head_dim)
    q, k, v = qkv.unbind(dim=2)
    if structured:
      a = sm_ops.structured_attention(q, k, v, padding_mask, causal, self.dropout_p, self.training)
    else:
      a = sm_ops.softmax_attention(q, k, v, mask, self.dropout_p, self.training)
    return dense_ops.linear(a.reshape(B, L, D), self.out, self.out_bias)


class TransformerBlock(nn.Module):
  def __init__(self, model_dim: int, intermediate_dim: int, num_heads: int, dropout: float = 0.0,
               activation: Callable = utils.gelu_approximate, layer_norm_epsilon: float = 1e-6,
               normalize_first: bool = True, causal: bool = False, init: Callable = _glorot_):
    super().__init__()
    self.attn = MultiHeadAttention(model_dim, num_heads, dropout, init)
    self.attn_norm_w, self.attn_norm_b = nn.Parameter(torch.ones(model_dim)), nn.Parameter(torch.zeros(model_dim))
    self.ffn_norm_w, self.ffn_norm_b = nn.Parameter(torch.ones(model_dim)), nn.Parameter(torch.zeros(model_dim))
    self.ffn_in = nn.Parameter(torch.empty(intermediate_dim, model_dim))
    self.ffn_in_bias = nn.Parameter(torch.zeros(intermediate_dim))
    self.ffn_out = nn.Parameter(torch.empty(model_dim, intermediate_dim))
    self.ffn_out_bias = nn.Parameter(torch.zeros(model_dim))
    init(self.ffn_in); init(self.ffn_out)
    self.activation, self.eps, self.normalize_first, self.causal = activation, layer_norm_epsilon, \
        normalize_first, causal
    self.attn_dropout, self.ffn_dropout = nn.Dropout(dropout), nn.Dropout(dropout)

  def forward(self, x, padding_mask=None, attention_mask=None):
    B, L, _ = x.shape
    mask = sm_ops.merge_masks(B, L, x.device, padding_mask=padding_mask, attention_mask=attention_mask,
                              causal=self.causal)
    ln = norm_ops.layer_norm
    kw = dict(padding_mask=padding_mask, causal=self.causal, structured=attention_mask is None)
    if self.normalize_first:
      x = x + self.attn_dropout(self.attn(ln(x, self.attn_norm_w, self.attn_norm_b, self.eps), mask, **kw)).to(x.dtype)
      h = self.activation(dense_ops.linear(ln(x, self.ffn_norm_w, self.ffn_norm_b, self.eps), self.ffn_in,
                                           self.ffn_in_bias))
      return x + self.ffn_dropout(dense_ops.linear(h, self.ffn_out, self.ffn_out_bias)).to(x.dtype)
    x = ln(x + self.attn_dropout(self.attn(x, mask, **kw)).to(x.dtype), self.attn_norm_w, self.attn_norm_b, self.eps)
    h = self.activation(dense_ops.linear(x, self.ffn_in, self.ffn_in_bias))
    return ln(x + self.ffn_dropout(dense_ops.linear(h, self.ffn_out, self.ffn_out_bias)).to(x.dtype),
              self.ffn_norm_w, self.ffn_norm_b, self.eps)
