"""SASRec: self-attentive sequential recommendation (`recml/layers/keras/sasrec.py:36-163`).
Item embedding (tied reverse) + learned positions → final_norm → dropout → N causal pre-LN
transformer blocks → final_norm → tied vocabulary logits."""
from __future__ import annotations

import math

import torch
from torch import nn

from recml_b200.layers import embeddings as emb_layers
from recml_b200.layers import utils as layer_utils
from recml_b200.layers import transformer
from recml_b200.ops import norm as norm_ops


class SASRec(layer_utils.Configurable, nn.Module):
  def __init__(self, *, vocab_size: int, max_positions: int, model_dim: int, mlp_dim: int, num_heads: int,
               num_layers: int, dropout: float = 0.0, norm_eps: float = 1e-6, scale_by_sqrt_dim: bool = False,
               add_head: bool = True):
    super().__init__()
    # vocab_size None: the caller owns the (sharded) item table and feeds embeddings to `encode_embeddings`
    self.item_embedding = (emb_layers.ReversibleEmbedding(vocab_size, model_dim, tie_weights=True)
                           if vocab_size is not None else None)
    self.position_embedding = emb_layers.PositionEmbedding(max_positions, model_dim)
    self.embeddings_dropout = nn.Dropout(dropout)
    self.decoder_blocks = nn.ModuleList(
        transformer.TransformerBlock(model_dim, mlp_dim, num_heads, dropout, layer_norm_epsilon=norm_eps,
                                     normalize_first=True, causal=True) for _ in range(num_layers))
    self.final_norm_w, self.final_norm_b = nn.Parameter(torch.ones(model_dim)), nn.Parameter(torch.zeros(model_dim))
    self.norm_eps, self.model_dim, self.scale_by_sqrt_dim, self.add_head = norm_eps, model_dim, \
        scale_by_sqrt_dim, add_head

  def compute_output_shape(self, inputs_shape):
    """Output shape for ids of `inputs_shape` (`recml/layers/keras/sasrec.py:165-167`)."""
    c = self.__dict__["_init_config"]
    return (*inputs_shape, c["vocab_size"] if c["add_head"] else c["model_dim"])

  def _norm(self, x):
    return norm_ops.layer_norm(x, self.final_norm_w, self.final_norm_b, self.norm_eps)

  def encode(self, inputs, padding_mask=None, attention_mask=None):
    """Sequence states `[B, L, D]` (what the sharded-vocabulary heads consume)."""
    return self.encode_embeddings(self.item_embedding(inputs), padding_mask, attention_mask)

  def encode_embeddings(self, e, padding_mask=None, attention_mask=None):
    """Same as `encode` for item embeddings `[B, L, D]` that were looked up elsewhere."""
    if self.scale_by_sqrt_dim:
      e = e * math.sqrt(self.model_dim)
    e = self.embeddings_dropout(self._norm(e + self.position_embedding(e)))
    for block in self.decoder_blocks:
      e = block(e, padding_mask=padding_mask, attention_mask=attention_mask)
    return self._norm(e)

  def forward(self, inputs, padding_mask=None, attention_mask=None):
    e = self.encode(inputs, padding_mask, attention_mask)
    return e if not self.add_head else self.item_embedding(e, reverse=True)
