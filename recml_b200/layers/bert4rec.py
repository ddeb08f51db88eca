"""BERT4Rec (`recml/layers/keras/bert4rec.py:37-208`): item + optional type + position embeddings
→ LN(eps 1e-12) → dropout → N post-LN encoder blocks → masked-LM head at `mask_positions`
(dense+gelu → LN → tied reverse embedding + vocabulary bias).  TruncatedNormal(0.02) inits."""
from __future__ import annotations

import torch
from torch import nn

from recml_b200.layers import embeddings as emb_layers
from recml_b200.layers import utils as layer_utils
from recml_b200.layers import transformer, utils
from recml_b200.ops import dense as dense_ops
from recml_b200.ops import norm as norm_ops


def _trunc02_(w):
  nn.init.trunc_normal_(w, 0.0, 0.02, -0.04, 0.04)


class MaskedLMHead(nn.Module):
  def __init__(self, token_embedding: emb_layers.ReversibleEmbedding, model_dim: int, vocab_size: int,
               activation=utils.gelu_approximate, eps: float = 1e-5):
    super().__init__()
    self.token_embedding = [token_embedding]   # not a sub-module: the weight is owned by the model
    self.dense = nn.Parameter(torch.empty(model_dim, model_dim))
    _trunc02_(self.dense)
    self.dense_bias = nn.Parameter(torch.zeros(model_dim))
    self.norm_w, self.norm_b = nn.Parameter(torch.ones(model_dim)), nn.Parameter(torch.zeros(model_dim))
    self.bias = nn.Parameter(torch.zeros(vocab_size))
    self.activation, self.eps = activation, eps

  def forward(self, x: torch.Tensor, mask_positions: torch.Tensor | None) -> torch.Tensor:
    if mask_positions is not None:
      x = torch.gather(x, 1, mask_positions.long()[..., None].expand(-1, -1, x.shape[-1]))
    h = self.activation(dense_ops.linear(x, self.dense, self.dense_bias))
    h = norm_ops.layer_norm(h, self.norm_w, self.norm_b, self.eps)
    return self.token_embedding[0](h, reverse=True).float() + self.bias


class BERT4Rec(layer_utils.Configurable, nn.Module):
  def __init__(self, *, vocab_size: int, max_positions: int, num_types: int | None = None, model_dim: int,
               mlp_dim: int, num_heads: int, num_layers: int, dropout: float = 0.0, norm_eps: float = 1e-12,
               add_head: bool = True):
    super().__init__()
    self.item_embedding = emb_layers.ReversibleEmbedding(vocab_size, model_dim, tie_weights=True, truncated=True)
    self.type_embedding = None
    if num_types is not None:
      self.type_embedding = nn.Embedding(num_types, model_dim)
      _trunc02_(self.type_embedding.weight)
    self.position_embedding = emb_layers.PositionEmbedding(max_positions, model_dim, truncated=True)
    self.embeddings_norm_w = nn.Parameter(torch.ones(model_dim))
    self.embeddings_norm_b = nn.Parameter(torch.zeros(model_dim))
    self.embeddings_dropout = nn.Dropout(dropout)
    self.encoder_blocks = nn.ModuleList(
        transformer.TransformerBlock(model_dim, mlp_dim, num_heads, dropout, layer_norm_epsilon=norm_eps,
                                     normalize_first=False, causal=False, init=_trunc02_)
        for _ in range(num_layers))
    self.head = MaskedLMHead(self.item_embedding, model_dim, vocab_size) if add_head else None

  def compute_output_shape(self, inputs_shape, mask_positions_shape=None):
    """Output shape for ids of `inputs_shape`; with the masked-LM head the rows are the masked positions
    (`recml/layers/keras/bert4rec.py:194-205`)."""
    c = self.__dict__["_init_config"]
    if c["add_head"]:
      if mask_positions_shape is None:
        raise ValueError("`mask_positions_shape` cannot be None when `add_head` is True.")
      return (*inputs_shape[:-1], mask_positions_shape[-1], c["vocab_size"])
    return (*inputs_shape, c["model_dim"])

  def forward(self, inputs, type_ids=None, padding_mask=None, attention_mask=None, mask_positions=None):
    e = self.item_embedding(inputs)
    if self.type_embedding is not None:
      if type_ids is None:
        raise ValueError("`type_ids` cannot be None when `num_types` is not None.")
      e = e + self.type_embedding(type_ids.long())
    e = e + self.position_embedding(e)
    e = self.embeddings_dropout(norm_ops.layer_norm(e, self.embeddings_norm_w, self.embeddings_norm_b, 1e-12))
    for block in self.encoder_blocks:
      e = block(e, padding_mask=padding_mask, attention_mask=attention_mask)
    if self.head is None:
      return e
    return self.head(e, mask_positions)
