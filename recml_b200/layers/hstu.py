"""HSTU — Hierarchical Sequential Transduction Unit (`recml/layers/keras/hstu.py:33-628`).

Block: n = LN(x); u, q, k, v = silu(n·W); a = pointwise-SiLU (or softmax) attention(q, k, v);
y = LN over (heads, head_dim)(a); out = (u ⊙ y)·W_o + x.  Model: item embedding (untied reverse
matrix) + optional learned positions → `final_norm` → dropout → blocks → `final_norm` again →
vocabulary logits.  Unlike the reference model, the relative position / time-bucket bias IS wired
into the blocks when `timestamps` / `use_relative_bias` are given (the reference builds the bias
layers but never passes them to the blocks).

Two execution forms share the parameters: the dense `[B, L, D]` form with explicit masks, and the
packed (jagged) form in which only real tokens exist — that is the one the B200 kernels serve.
"""
from __future__ import annotations

import math
from typing import Callable

import torch
from torch import nn

from recml_b200.layers import embeddings as emb_layers
from recml_b200.layers import utils as layer_utils
from recml_b200.layers import utils
from recml_b200.ops import dense as dense_ops
from recml_b200.ops import hstu_attention as attn_ops
from recml_b200.ops import norm as norm_ops


def default_bucketization(tensor: torch.Tensor, bucket_size: float = 0.301) -> torch.Tensor:
  v = tensor.abs().clamp(min=1, max=int(1e9)).to(torch.float32)
  return (torch.log(v) / bucket_size).to(torch.int64)


class RelativePositionalBias(layer_utils.Configurable, nn.Module):
  """2N−1 learned scalars expanded to a Toeplitz `[1, n, n]` bias: bias[i, j] = w[(j − i) + n − 1]."""

  def __init__(self, max_seq_len: int, init_std: float = 0.02):
    super().__init__()
    self.pos_biases = nn.Parameter(torch.empty(2 * max_seq_len - 1))
    nn.init.normal_(self.pos_biases, 0.0, init_std)

  def forward(self, inputs: torch.Tensor) -> torch.Tensor:
    n = inputs.shape[-1]
    w = self.pos_biases[:2 * n - 1]
    i = torch.arange(n, device=w.device)
    return w[(i[None, :] - i[:, None]) + n - 1][None]


class RelativeBucketedTimeAndPositionBasedBias(layer_utils.Configurable, nn.Module):
  """ts_w[bucket(t_ext[i+1] − t[j])] (+ positional bias); `[B, N] → [B, N, N]`."""

  def __init__(self, num_buckets: int = 128, bucketization_fn: Callable = default_bucketization,
               position_bias_layer: nn.Module | None = None, init_std: float = 0.02):
    super().__init__()
    self.num_buckets = num_buckets
    self.bucketization_fn = bucketization_fn
    self.positional_bias = position_bias_layer
    self.ts_w = nn.Parameter(torch.empty(num_buckets + 1))
    nn.init.normal_(self.ts_w, 0.0, init_std)

  def time_bias(self, inputs: torch.Tensor) -> torch.Tensor:
    ext = torch.cat([inputs, inputs[:, -1:]], dim=1)
    delta = ext[:, 1:, None] - ext[:, None, :-1]
    buckets = torch.clamp(self.bucketization_fn(delta), 0, self.num_buckets)
    return self.ts_w[buckets]

  def forward(self, inputs: torch.Tensor) -> torch.Tensor:
    tb = self.time_bias(inputs)
    return tb if self.positional_bias is None else self.positional_bias(inputs) + tb


def _glorot_uniform_(w: torch.Tensor, fan_in: int, fan_out: int) -> None:
  lim = math.sqrt(6.0 / (fan_in + fan_out))
  nn.init.uniform_(w, -lim, lim)


class HSTUBlock(layer_utils.Configurable, nn.Module):
  def __init__(self, model_dim: int, num_heads: int, use_bias: bool = False, activation=torch.nn.functional.silu,
               layer_norm_epsilon: float = 1e-6, scaled_pointwise_attn: bool = False,
               softmax_attention: bool = False, dropout: float = 0.0):
    super().__init__()
    assert model_dim % num_heads == 0
    self.model_dim, self.num_heads, self.head_dim = model_dim, num_heads, model_dim // num_heads
    self.eps, self.scaled, self.softmax, self.dropout_p = layer_norm_epsilon, scaled_pointwise_attn, \
        softmax_attention, dropout
    self.activation = activation
    self.input_norm_w = nn.Parameter(torch.ones(model_dim))
    self.input_norm_b = nn.Parameter(torch.zeros(model_dim))
    # u, q, k, v projections fused into one [4D, D] weight (rows: u | q | k | v, each [H·Dh])
    self.uqkv = nn.Parameter(torch.empty(4 * model_dim, model_dim))
    for i in range(4):
      _glorot_uniform_(self.uqkv.data[i * model_dim:(i + 1) * model_dim], model_dim, model_dim)
    self.uqkv_bias = nn.Parameter(torch.zeros(4 * model_dim)) if use_bias else None
    self.attn_norm_w = nn.Parameter(torch.ones(num_heads, self.head_dim))
    self.attn_norm_b = nn.Parameter(torch.zeros(num_heads, self.head_dim))
    self.out = nn.Parameter(torch.empty(model_dim, model_dim))
    _glorot_uniform_(self.out, model_dim, model_dim)
    self.out_bias = nn.Parameter(torch.zeros(model_dim)) if use_bias else None

  def _project(self, x):
    n = norm_ops.layer_norm(x, self.input_norm_w, self.input_norm_b, self.eps)
    h = self.activation(dense_ops.linear(n, self.uqkv, self.uqkv_bias))
    return h.reshape(*x.shape[:-1], 4, self.num_heads, self.head_dim).unbind(dim=-3)

  def _finish(self, x, u, attn):
    y = norm_ops.layer_norm(attn, self.attn_norm_w, self.attn_norm_b, self.eps, gate=u, norm_dims=2)
    y = y.reshape(*x.shape[:-1], self.model_dim)
    return dense_ops.linear(y, self.out, self.out_bias, residual=x).to(x.dtype)

  def forward(self, inputs: torch.Tensor, attention_mask: torch.Tensor, attention_bias: torch.Tensor | None = None):
    """Dense form: inputs `[B, L, D]`, mask / bias `[B, L, L]`."""
    u, q, k, v = self._project(inputs)
    if self.softmax:
      qs = q.float() / math.sqrt(self.head_dim)
      s = torch.einsum("bthd,bshd->bhts", qs, k.float())
      if attention_bias is not None:
        s = s + attention_bias[:, None].float()
      s = torch.where(attention_mask[:, None].bool(), s,
                      torch.full_like(s, utils.large_negative_for_attention(s.dtype)))
      p = torch.softmax(s, dim=-1)
      if self.training and self.dropout_p > 0:
        p = torch.nn.functional.dropout(p, self.dropout_p)
      attn = torch.einsum("bhts,bshd->bthd", p, v.float()).to(inputs.dtype)
    else:
      attn = attn_ops.pointwise_attention_dense(q, k, v, attention_mask, attention_bias, scaled=self.scaled,
                                                dropout_p=self.dropout_p, training=self.training)
    return self._finish(inputs, u, attn)

  def forward_jagged(self, tokens: torch.Tensor, seq_offsets: torch.Tensor, max_seq_len: int, *,
                     pos_w=None, ts_w=None, timestamps=None, segment_ids=None, row_mask=None):
    """Packed form: tokens `[T, D]`; causal pointwise attention inside every sequence.  `segment_ids [T]`
    restricts a query to keys of its own segment; `row_mask [T]` zeroes the attention output of the rows
    where it is 0 (padded positions of a dense batch that is run through the packed kernels)."""
    scale = 1.0 / math.sqrt(self.head_dim) if self.scaled else 1.0
    z = None
    if self.activation is torch.nn.functional.silu and tokens.is_cuda:
      n = norm_ops.layer_norm(tokens, self.input_norm_w, self.input_norm_b, self.eps)
      z = dense_ops.linear(n, self.uqkv, self.uqkv_bias)
    if z is not None and attn_ops.fused_block_ok(z, self.head_dim):
      # activation, split and attention as one autograd node: see `silu_split_attention`
      u, attn = attn_ops.silu_split_attention(z, self.num_heads, seq_offsets, max_seq_len, pos_w=pos_w, ts_w=ts_w,
                                              timestamps=timestamps, causal=True, scale=scale,
                                              segment_ids=segment_ids,
                                              dropout_p=self.dropout_p if self.training else 0.0)
    else:
      if z is not None:
        u, q, k, v = self.activation(z).reshape(*tokens.shape[:-1], 4, self.num_heads, self.head_dim).unbind(dim=-3)
      else:
        u, q, k, v = self._project(tokens)
      attn = attn_ops.jagged_pointwise_attention(q, k, v, seq_offsets, max_seq_len, pos_w=pos_w, ts_w=ts_w,
                                                 timestamps=timestamps, causal=True, scale=scale,
                                                 segment_ids=segment_ids,
                                                 dropout_p=self.dropout_p if self.training else 0.0)
    if row_mask is not None:
      attn = attn * row_mask[:, None, None].to(attn.dtype)
    return self._finish(tokens, u, attn)


class HSTU(layer_utils.Configurable, nn.Module):
  def __init__(self, *, vocab_size: int, max_positions: int | None = None, model_dim: int, num_heads: int,
               num_layers: int, dropout: float = 0.0, norm_eps: float = 1e-6, scale_by_sqrt_dim: bool = False,
               add_head: bool = True, use_relative_bias: bool = False, num_time_buckets: int = 128,
               max_seq_len: int | None = None):
    super().__init__()
    # vocab_size None: the caller owns the item table (e.g. a sharded embedding) and feeds embeddings
    self.item_embedding = (emb_layers.ReversibleEmbedding(vocab_size, model_dim, tie_weights=False)
                           if vocab_size is not None else None)
    self.position_embedding = (emb_layers.PositionEmbedding(max_positions, model_dim)
                               if max_positions is not None else None)
    self.embeddings_dropout = nn.Dropout(dropout)
    self.decoder_blocks = nn.ModuleList(
        HSTUBlock(model_dim, num_heads, dropout=dropout, layer_norm_epsilon=norm_eps) for _ in range(num_layers))
    self.final_norm_w = nn.Parameter(torch.ones(model_dim))
    self.final_norm_b = nn.Parameter(torch.zeros(model_dim))
    self.norm_eps, self.model_dim, self.scale_by_sqrt_dim, self.add_head = norm_eps, model_dim, \
        scale_by_sqrt_dim, add_head
    self.max_seq_len = max_seq_len or max_positions
    self.relative_bias = None
    if use_relative_bias:
      assert self.max_seq_len is not None, "relative bias needs max_seq_len"
      self.relative_bias = RelativeBucketedTimeAndPositionBasedBias(
          num_time_buckets, position_bias_layer=RelativePositionalBias(self.max_seq_len))

  def compute_output_shape(self, inputs_shape):
    """Output shape for ids of `inputs_shape` (`recml/layers/keras/hstu.py:623-625`)."""
    c = self.__dict__["_init_config"]
    return (*inputs_shape, c["vocab_size"] if c["add_head"] else c["model_dim"])

  def _final_norm(self, x):
    return norm_ops.layer_norm(x, self.final_norm_w, self.final_norm_b, self.norm_eps)

  def _embed(self, ids, positions=None):
    e = self.item_embedding(ids)
    if self.scale_by_sqrt_dim:
      e = e * math.sqrt(self.model_dim)
    if self.position_embedding is not None:
      e = e + self.position_embedding(e, positions)
    return self.embeddings_dropout(self._final_norm(e))

  def forward(self, inputs: torch.Tensor, padding_mask: torch.Tensor | None = None,
              attention_mask: torch.Tensor | None = None, timestamps: torch.Tensor | None = None):
    """Dense form (reference call signature): inputs `[B, L]` ids → logits `[B, L, V]`."""
    e = self._embed(inputs)
    if attention_mask is None:
      if padding_mask is None:
        raise ValueError("Either `attention_mask` or `padding_mask` must be set.")
      if self._packed_kernels_apply(e):
        return self._forward_dense_through_packed_kernels(e, padding_mask, timestamps)
      attention_mask = utils.make_causal_mask(padding_mask)
    bias = None
    if self.relative_bias is not None:
      ts = timestamps if timestamps is not None else torch.zeros_like(inputs)
      bias = self.relative_bias(ts)
    for block in self.decoder_blocks:
      e = block(e, attention_mask, bias)
    e = self._final_norm(e)
    return e if not self.add_head else self.item_embedding(e, reverse=True)

  def _packed_kernels_apply(self, e: torch.Tensor) -> bool:
    """The dense (padded) call can run on the packed attention kernels: CUDA, head dim 64 / 128, SiLU
    attention (attention-weight dropout included) and, when there is a relative bias, a position table made for
    this padded length."""
    b = self.decoder_blocks[0]
    if not e.is_cuda or b.head_dim not in (64, 128) or b.softmax or b.scaled:
      return False
    return self.relative_bias is None or self.max_seq_len == e.shape[1]

  def _forward_dense_through_packed_kernels(self, e, padding_mask, timestamps):
    """`[B, L, D]` padded batch as B packed sequences of length L: the mask `valid[i] & valid[j] & (j <= i)` of
    the dense formulation becomes causality plus segment ids (every padded position is a segment of its own)
    plus zeroing the padded query rows; the normaliser is L in both."""
    B, L, D = e.shape
    dev = e.device
    valid = padding_mask.reshape(-1) != 0
    pos = torch.arange(B * L, device=dev, dtype=torch.int32)
    seg = torch.where(valid, torch.zeros_like(pos), -1 - pos)
    offs = torch.arange(B + 1, device=dev, dtype=torch.int32) * L
    pos_w = ts_w = None
    ts = None
    if self.relative_bias is not None:
      pos_w, ts_w = self.relative_bias.positional_bias.pos_biases, self.relative_bias.ts_w
      ts = (timestamps if timestamps is not None else torch.zeros(B, L, device=dev, dtype=torch.int64)).reshape(-1)
    x = e.reshape(B * L, D)
    for block in self.decoder_blocks:
      x = block.forward_jagged(x, offs, L, pos_w=pos_w, ts_w=ts_w, timestamps=ts, segment_ids=seg, row_mask=valid)
    x = self._final_norm(x).reshape(B, L, D)
    return x if not self.add_head else self.item_embedding(x, reverse=True)

  def forward_jagged(self, ids: torch.Tensor, seq_offsets: torch.Tensor, timestamps: torch.Tensor | None = None):
    """Packed form: ids `[T]`, `seq_offsets [B+1]` → token states `[T, D]` (heads are applied by the
    caller: sampled softmax or full-vocabulary scoring never materialise `[T, V]`)."""
    lens = seq_offsets[1:] - seq_offsets[:-1]
    positions = torch.arange(ids.numel(), device=ids.device) - torch.repeat_interleave(seq_offsets[:-1], lens)
    e = self._embed(ids, positions if self.position_embedding is not None else None)
    return self.encode_jagged(e, seq_offsets, timestamps)

  def encode_jagged(self, e: torch.Tensor, seq_offsets: torch.Tensor, timestamps: torch.Tensor | None = None,
                    normalize_input: bool = False):
    """Packed token embeddings `[T, D]` (already looked up) → token states `[T, D]`."""
    if normalize_input:
      e = self.embeddings_dropout(self._final_norm(e))
    pos_w = ts_w = None
    if self.relative_bias is not None:
      pos_w, ts_w = self.relative_bias.positional_bias.pos_biases, self.relative_bias.ts_w
    for block in self.decoder_blocks:
      e = block.forward_jagged(e, seq_offsets, self.max_seq_len, pos_w=pos_w, ts_w=ts_w, timestamps=timestamps)
    return self._final_norm(e)
