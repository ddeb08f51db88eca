"""Mamba2 / Mamba4Rec (`recml/layers/keras/mamba.py:149-752`).

Mamba2: z, xBC, dt projections → depthwise causal conv (k = d_conv) + SiLU on xBC →
dt = softplus(dt + dt_bias), A = −exp(a_log) → y = SSD(x·dt, A·dt, B, C) → RMS-scaled LN of
y ⊙ silu(z) → output projection.  Block: x1 = LN(drop(ssm(x)) + x); y = LN(FFN(x1) + x1), FFN =
Dense(d·ffn_expand, exact gelu) → drop → Dense(d) → drop; padded positions are zeroed."""
from __future__ import annotations

import math

import torch
from torch import nn

from recml_b200.layers import embeddings as emb_layers
from recml_b200.layers import utils as layer_utils
from recml_b200.ops import dense as dense_ops
from recml_b200.ops import norm as norm_ops
from recml_b200.ops import ssd as ssd_ops

segsum_chunked = ssd_ops.ssd_chunked


class Mamba2(layer_utils.Configurable, nn.Module):
  def __init__(self, d_model: int, d_state: int = 64, d_conv: int = 4, conv_init: float | None = None,
               expand: int = 4, nheads: int = 8, chunk_size: int = 256, init_range_a=(1, 16), dt_min: float = 0.001,
               dt_max: float = 0.1, dt_init_floor: float = 1e-4, dt_limit=(0.0, float("inf")),
               learn_init_states: bool = False, activation: str = "swish", use_dense_bias: bool = False,
               use_conv_bias: bool = False):
    super().__init__()
    assert activation in ("silu", "swish")
    self.d_model, self.d_state, self.d_conv, self.expand = d_model, d_state, d_conv, expand
    self.d_inner = expand * d_model
    self.nheads, self.ngroups, self.chunk_size = nheads, 1, chunk_size
    self.headdim = self.d_inner // nheads
    conv_dim = self.d_inner + 2 * self.ngroups * d_state
    mk = lambda o, i: nn.Parameter(nn.init.xavier_uniform_(torch.empty(o, i)))
    self.z_proj = mk(self.d_inner, d_model)
    self.xbc_proj = mk(conv_dim, d_model)
    self.dt_proj = mk(nheads, d_model)
    self.z_bias = nn.Parameter(torch.zeros(self.d_inner)) if use_dense_bias else None
    self.xbc_bias = nn.Parameter(torch.zeros(conv_dim)) if use_dense_bias else None
    self.dt_proj_bias = nn.Parameter(torch.zeros(nheads)) if use_dense_bias else None
    w = torch.empty(conv_dim, d_conv)
    if conv_init is None:
      lim = math.sqrt(6.0 / (d_conv + d_conv * conv_dim))
      w.uniform_(-lim, lim)
    else:
      w.uniform_(-conv_init, conv_init)
    self.conv_weight = nn.Parameter(w)
    self.conv_bias = nn.Parameter(torch.zeros(conv_dim)) if use_conv_bias else None
    # dt bias: inverse softplus of dt ~ logU(dt_min, dt_max), floored
    dt = torch.exp(torch.rand(nheads) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).clamp(min=dt_init_floor)
    self.dt_bias = nn.Parameter(dt + torch.log(-torch.expm1(-dt)))
    self.a_log = nn.Parameter(torch.log(torch.empty(nheads).uniform_(*init_range_a)))
    self.init_states = nn.Parameter(torch.zeros(nheads, self.headdim, d_state)) if learn_init_states else None
    self.norm_w = nn.Parameter(torch.ones(self.d_inner))
    self.norm_b = nn.Parameter(torch.zeros(self.d_inner))
    self.out_proj = mk(d_model, self.d_inner)
    self.out_bias = nn.Parameter(torch.zeros(d_model)) if use_dense_bias else None
    self.dt_limit = dt_limit

  def forward(self, inputs: torch.Tensor) -> torch.Tensor:
    B, L, _ = inputs.shape
    a = -torch.exp(self.a_log.float())
    z = dense_ops.linear(inputs, self.z_proj, self.z_bias)
    xbc = dense_ops.linear(inputs, self.xbc_proj, self.xbc_bias)
    dt = torch.nn.functional.softplus(dense_ops.linear(inputs, self.dt_proj, self.dt_proj_bias).float() + self.dt_bias)
    xbc = ssd_ops.conv1d_silu(xbc, self.conv_weight, self.conv_bias)
    x, b, c = torch.split(xbc.float(), [self.d_inner, self.d_state, self.d_state], dim=-1)
    x = x.reshape(B, L, self.nheads, self.headdim)
    b = b.reshape(B, L, 1, self.d_state)
    c = c.reshape(B, L, 1, self.d_state)
    xs, as_ = x * dt[..., None], a * dt
    y = ssd_ops.ssd_scan(xs, as_, b, c, self.chunk_size, self.init_states)
    y = y.reshape(B, L, self.d_inner)
    y = norm_ops.layer_norm((y * torch.nn.functional.silu(z.float())).to(inputs.dtype), self.norm_w, self.norm_b,
                            1e-5, rms=True)
    return dense_ops.linear(y, self.out_proj, self.out_bias)


class Mamba2Block(layer_utils.Configurable, nn.Module):
  def __init__(self, d_model: int, d_state: int = 64, d_conv: int = 4, expand: int = 2, nheads: int = 8,
               chunk_size: int = 64, ffn_expand: int = 12, norm_eps: float = 1e-12, dropout: float = 0.0):
    super().__init__()
    self.mamba_ssm = Mamba2(d_model, d_state, d_conv, expand=expand, nheads=nheads, chunk_size=chunk_size)
    self.ln_w, self.ln_b = nn.Parameter(torch.ones(d_model)), nn.Parameter(torch.zeros(d_model))
    self.final_ln_w, self.final_ln_b = nn.Parameter(torch.ones(d_model)), nn.Parameter(torch.zeros(d_model))
    self.ffn_in = nn.Parameter(nn.init.xavier_uniform_(torch.empty(d_model * ffn_expand, d_model)))
    self.ffn_in_bias = nn.Parameter(torch.zeros(d_model * ffn_expand))
    self.ffn_out = nn.Parameter(nn.init.xavier_uniform_(torch.empty(d_model, d_model * ffn_expand)))
    self.ffn_out_bias = nn.Parameter(torch.zeros(d_model))
    self.norm_eps = norm_eps
    self.mamba_dropout, self.drop1, self.drop2 = nn.Dropout(dropout), nn.Dropout(dropout), nn.Dropout(dropout)

  def forward(self, inputs, padding_mask=None):
    x = self.mamba_dropout(self.mamba_ssm(inputs)).to(inputs.dtype)
    x = norm_ops.layer_norm(x + inputs, self.ln_w, self.ln_b, 1e-12)
    h = self.drop1(torch.nn.functional.gelu(dense_ops.linear(x, self.ffn_in, self.ffn_in_bias)))
    y = self.drop2(dense_ops.linear(h, self.ffn_out, self.ffn_out_bias)).to(x.dtype)
    y = norm_ops.layer_norm(y + x, self.final_ln_w, self.final_ln_b, self.norm_eps)
    if padding_mask is not None:
      y = torch.where(padding_mask.bool()[..., None], y, torch.zeros_like(y))
    return y


class Mamba2Stack(layer_utils.Configurable, nn.Module):
  def __init__(self, num_layers: int, **block_kwargs):
    super().__init__()
    self.blocks = nn.ModuleList(Mamba2Block(**block_kwargs) for _ in range(num_layers))

  def forward(self, x, padding_mask=None):
    for blk in self.blocks:
      x = blk(x, padding_mask)
    return x


class Mamba4Rec(layer_utils.Configurable, nn.Module):
  def __init__(self, vocab_size: int, model_dim: int, mlp_expand: int, num_heads: int, num_layers: int,
               d_expand: int, d_state: int = 64, d_conv: int = 4, chunk_size: int = 256, norm_eps: float = 1e-6,
               dropout: float = 0.0, add_head: bool = True):
    super().__init__()
    self.item_embedding = emb_layers.ReversibleEmbedding(vocab_size, model_dim, tie_weights=True)
    self.dropout_layer = nn.Dropout(dropout)
    self.emb_norm_w, self.emb_norm_b = nn.Parameter(torch.ones(model_dim)), nn.Parameter(torch.zeros(model_dim))
    self.decoder_blocks = nn.ModuleList(
        Mamba2Block(model_dim, d_state, d_conv, expand=d_expand, nheads=num_heads, ffn_expand=mlp_expand,
                    chunk_size=chunk_size, norm_eps=norm_eps, dropout=dropout) for _ in range(num_layers))
    self.norm_eps, self.add_head = norm_eps, add_head

  def compute_output_shape(self, inputs_shape):
    """Output shape for ids of `inputs_shape` (`recml/layers/keras/mamba.py:747-749`)."""
    c = self.__dict__["_init_config"]
    return (*inputs_shape, c["vocab_size"] if c["add_head"] else c["model_dim"])

  def forward(self, inputs, padding_mask=None):
    x = self.dropout_layer(self.item_embedding(inputs))
    x = norm_ops.layer_norm(x, self.emb_norm_w, self.emb_norm_b, self.norm_eps)
    for blk in self.decoder_blocks:
      x = blk(x, padding_mask)
    return x if not self.add_head else self.item_embedding(x, reverse=True)
