"""Embedding layers used by the sequence models: `ReversibleEmbedding` (lookup + tied / untied
reverse projection to vocabulary logits) and `PositionEmbedding` (learned positions), restating
the keras_hub layers the reference builds on (`recml/layers/keras/hstu.py:521-537`,
`sasrec.py:69-83`)."""
from __future__ import annotations

import torch
from torch import nn

from recml_b200.ops import dense as dense_ops


class ReversibleEmbedding(nn.Module):
  def __init__(self, input_dim: int, output_dim: int, tie_weights: bool = True, init_std: float = 0.02,
               truncated: bool = False):
    super().__init__()
    self.embeddings = nn.Parameter(torch.empty(input_dim, output_dim))
    self.tie_weights = tie_weights
    init = (lambda t: nn.init.trunc_normal_(t, 0.0, init_std, -2 * init_std, 2 * init_std)) if truncated \
        else (lambda t: nn.init.normal_(t, 0.0, init_std))
    init(self.embeddings)
    if not tie_weights:
      self.reverse_embeddings = nn.Parameter(torch.empty(output_dim, input_dim))
      init(self.reverse_embeddings)

  def forward(self, inputs: torch.Tensor, reverse: bool = False) -> torch.Tensor:
    if not reverse:
      return torch.nn.functional.embedding(inputs.long(), self.embeddings)
    if self.tie_weights:
      return dense_ops.linear(inputs, self.embeddings)             # x·Eᵀ
    return dense_ops.linear(inputs, self.reverse_embeddings.t().contiguous()
                            if not inputs.is_cuda else self.reverse_embeddings.t())

  def reverse_matrix(self) -> torch.Tensor:
    """`[V, D]` matrix whose rows score the items (E, or Rᵀ when untied)."""
    return self.embeddings if self.tie_weights else self.reverse_embeddings.t()


class PositionEmbedding(nn.Module):
  def __init__(self, sequence_length: int, dim: int, init_std: float = 0.02, truncated: bool = False):
    super().__init__()
    self.position_embeddings = nn.Parameter(torch.empty(sequence_length, dim))
    if truncated:
      nn.init.trunc_normal_(self.position_embeddings, 0.0, init_std, -2 * init_std, 2 * init_std)
    else:
      nn.init.normal_(self.position_embeddings, 0.0, init_std)

  def forward(self, inputs: torch.Tensor, positions: torch.Tensor | None = None) -> torch.Tensor:
    """Position rows broadcast against `[..., L, D]` inputs (or gathered at explicit positions)."""
    if positions is not None:
      return self.position_embeddings[positions.long()]
    return self.position_embeddings[:inputs.shape[-2]].to(inputs.dtype)
