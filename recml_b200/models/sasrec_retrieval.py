"""SASRec with a row-sharded item table: BCE training on one positive and one sampled negative per
position, full-vocabulary evaluation (NDCG@10 / Recall@10 / MRR) through the sharded rank kernel.
Reference model: `recml/layers/keras/sasrec.py:36-163` (dense tied embedding + `[B, L, V]` logits)."""
from __future__ import annotations

import torch
from torch import nn

from recml_b200 import embedding as emb
from recml_b200.layers import sasrec as sasrec_layers
from recml_b200.ops import vocab_rank


class SASRecRetrieval(nn.Module):
  def __init__(self, *, vocab_size: int, max_positions: int = 200, model_dim: int = 256, mlp_dim: int = 1024,
               num_heads: int = 4, num_layers: int = 2, dropout: float = 0.0, batch_size: int,
               embedding_optimizer: emb.OptimizerSpec | None = None, device=None, group=None, backend: str = "auto",
               seed: int = 0):
    super().__init__()
    self.vocab_size, self.model_dim, self.max_positions, self.batch_size = vocab_size, model_dim, max_positions, batch_size
    self.group = group
    init = emb.specs.normal_init(0.02)
    mk = lambda: emb.EmbeddingSpec(vocab_size, model_dim, combiner="sum", initializer=init, table_name="items")
    self.items = emb.ShardedEmbedding(
        emb.ShardedEmbeddingConfig({"input": mk(), "positive": mk(), "negative": mk()},
                                   embedding_optimizer or emb.RowWiseAdagradOptimizerSpec(0.01),
                                   sharding_strategy="MOD", backend=backend, seed=seed), device=device, group=group)
    self.encoder = sasrec_layers.SASRec(vocab_size=None, max_positions=max_positions, model_dim=model_dim,
                                        mlp_dim=mlp_dim, num_heads=num_heads, num_layers=num_layers, dropout=dropout,
                                        add_head=False)
    if device is not None:
      self.encoder.to(device)
    self._ranker = None
    self._shadow = None

  def _lookup(self, a, b, c):
    B, L = a.shape
    kjt = emb.KeyedJagged.from_dense({"input": a.reshape(-1, 1), "positive": b.reshape(-1, 1),
                                      "negative": c.reshape(-1, 1)}).to_device(a.device)
    out = self.items(kjt)                       # [B·L, 3, D]
    return out.view(B, L, 3, self.model_dim).unbind(dim=2)

  def forward(self, input_ids, positive_ids, negative_ids, padding_mask):
    """All `[B, L]`.  Returns the masked mean BCE over positions."""
    e_in, e_pos, e_neg = self._lookup(input_ids, positive_ids, negative_ids)
    h = self.encoder.encode_embeddings(e_in, padding_mask).float()
    pos, neg = (h * e_pos.float()).sum(-1), (h * e_neg.float()).sum(-1)
    w = padding_mask.float()
    loss = (torch.nn.functional.softplus(-pos) + torch.nn.functional.softplus(neg)) * w
    return loss.sum() / w.sum().clamp_min(1.0)

  @torch.no_grad()
  def item_shard_bf16(self):
    """bf16 copy of this rank's rows of the item table and the local-row → global-id map (MOD layout)."""
    tp = self.items.plan.tables["items"]
    w = self.items.stack_weights[tp.stack][tp.row_base:tp.row_base + tp.local_rows]
    if self._shadow is None or self._shadow.shape != w.shape:
      self._shadow = torch.empty(w.shape, dtype=torch.bfloat16, device=w.device)
    self._shadow.copy_(w)
    W, rank = self.items.world, self.items.rank
    if tp.placement is emb.Placement.ROW_WISE:
      return self._shadow, W, (rank - tp.rotation) % W
    return self._shadow, 1, 0

  @torch.no_grad()
  def evaluate_ranks(self, input_ids, padding_mask, target_ids):
    """1-based full-vocabulary rank of `target_ids [B]` given the history (last valid position)."""
    B, L = input_ids.shape
    zeros = torch.zeros_like(input_ids)
    tgt_col = target_ids.view(B, 1).expand(B, L).contiguous()
    e_in, e_tgt, _ = self._lookup(input_ids, tgt_col, zeros)
    h = self.encoder.encode_embeddings(e_in, padding_mask)
    last = (padding_mask.long() * torch.arange(L, device=input_ids.device)).argmax(dim=1)
    h_last = h[torch.arange(B, device=h.device), last].to(torch.bfloat16)
    pos = (h_last.float() * e_tgt[:, 0].to(torch.bfloat16).float()).sum(-1)
    if self._ranker is None:
      self._ranker = vocab_rank.VocabRanker(B, self.model_dim, self.group, input_ids.device)
    shard, mul, add = self.item_shard_bf16()
    tp = self.items.plan.tables["items"]
    if tp.placement is emb.Placement.TABLE_WISE and self.items.world > 1 and self.items.rank != tp.owner:
      shard = shard[:0]
    return self._ranker.ranks(h_last, pos, target_ids, shard.contiguous(), mul, add)
