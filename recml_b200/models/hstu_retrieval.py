"""HSTU generative retrieval with a sharded item table and sampled-softmax training.

The reference trains HSTU with a dense `[V, D]` embedding and a full-vocabulary softmax on the last
position (`recml/examples/train_hstu_jax.py:98-236`, vocab 5 M, length 50).  For a 10 M × 256 item
table on 8 GPUs the table is row-sharded (`recml_b200.embedding`), sequences are packed (jagged) and
every position predicts its next item against 1 positive + `num_negatives` shared uniform negatives
+ `num_in_batch` in-batch negatives (other positions' targets), so no `[T, V]` logits ever exist.
"""
from __future__ import annotations

import torch
from torch import nn

from recml_b200 import embedding as emb
from recml_b200.layers import hstu as hstu_layers
from recml_b200.ops import dense as dense_ops
from recml_b200.ops import norm as norm_ops
from recml_b200.ops import sampled_softmax


class HSTURetrieval(nn.Module):
  def __init__(self, *, vocab_size: int, model_dim: int = 256, num_heads: int = 4, num_layers: int = 8,
               max_seq_len: int = 4096, token_capacity: int, num_negatives: int = 512, num_in_batch: int = 512,
               dropout: float = 0.0, embedding_optimizer: emb.OptimizerSpec | None = None, device=None, group=None,
               backend: str = "auto", seed: int = 0, temperature: float = 0.05):
    super().__init__()
    self.token_capacity, self.num_negatives, self.num_in_batch = token_capacity, num_negatives, num_in_batch
    self.model_dim, self.temperature = model_dim, temperature
    init = emb.specs.normal_init(0.02)
    mk = lambda: emb.EmbeddingSpec(vocab_size, model_dim, combiner="sum", initializer=init, table_name="items")
    # three views of ONE table: input items, target items, shared negatives (bags of size 0 or 1)
    self.items = emb.ShardedEmbedding(
        emb.ShardedEmbeddingConfig({"input": mk(), "target": mk(), "negative": mk()},
                                   embedding_optimizer or emb.RowWiseAdagradOptimizerSpec(0.01),
                                   sharding_strategy="MOD", backend=backend, seed=seed), device=device, group=group)
    self._unit_w: dict = {}
    self.encoder = hstu_layers.HSTU(vocab_size=None, model_dim=model_dim, num_heads=num_heads,
                                    num_layers=num_layers, dropout=dropout, use_relative_bias=True,
                                    max_seq_len=max_seq_len)
    if device is not None:
      self.encoder.to(device)

  def _unit_rows(self, x: torch.Tensor) -> torch.Tensor:
    """Rows scaled to unit L2 norm.  On CUDA this is the fused RMS-norm kernel pair (x / sqrt(mean(x^2)) with the
    constant weight 1 / sqrt(D)): one pass forward and one backward instead of a chain of fp32 element-wise
    kernels over `[T, D]`."""
    D = x.shape[-1]
    if x.is_cuda and x.dtype == torch.bfloat16 and D % 8 == 0:
      w = self._unit_w.get((D, x.device))
      if w is None:
        w = self._unit_w[(D, x.device)] = torch.full((D,), D ** -0.5, dtype=torch.float32, device=x.device)
      return norm_ops.layer_norm(x, w, None, 1e-24, rms=True)
    return torch.nn.functional.normalize(x.float(), dim=-1)

  def make_lookup_batch(self, input_ids, target_ids, negative_ids) -> emb.KeyedJagged:
    """One jagged batch of `token_capacity` rows: row t carries input / target id of token t (none
    for padding rows) and row n < num_negatives carries negative n."""
    cap, dev = self.token_capacity, input_ids.device
    T, N = input_ids.numel(), negative_ids.numel()
    ar = torch.arange(cap + 1, device=dev, dtype=torch.int32)
    o_in = torch.clamp(ar, max=T)
    o_tg = T + torch.clamp(ar, max=T)
    o_ng = 2 * T + torch.clamp(ar, max=N)
    offsets = torch.cat([o_in[:-1], o_tg[:-1], o_ng])
    values = torch.cat([input_ids, target_ids, negative_ids]).to(torch.int32)
    return emb.KeyedJagged(("input", "target", "negative"), values, offsets, None, cap)

  def forward(self, input_ids, target_ids, negative_ids, seq_offsets, timestamps, target_weights):
    """Packed batch: ids `[T]`, `seq_offsets [B+1]`, timestamps `[T]`, weights `[T]` (0 where a position
    has no next item).  Returns (mean loss, hit@1 among the sampled candidates)."""
    T = input_ids.numel()
    looked = self.items(self.make_lookup_batch(input_ids, target_ids, negative_ids))   # [cap, 3, D]
    e_in, e_tg, e_ng = looked[:T, 0], looked[:T, 1], looked[:self.num_negatives, 2]
    h = self.encoder.encode_jagged(e_in, seq_offsets, timestamps, normalize_input=True)   # [T, D]
    h = self._unit_rows(h).to(e_in.dtype)
    stride = max(T // max(self.num_in_batch, 1), 1)
    inb_idx = torch.arange(0, T, stride, device=input_ids.device)[:self.num_in_batch]
    cand = torch.cat([e_ng, e_tg[inb_idx]], dim=0)
    cand = self._unit_rows(cand).to(h.dtype)
    cand_ids = torch.cat([negative_ids, target_ids[inb_idx]])
    pos = (h.float() * self._unit_rows(e_tg).float()).sum(-1)
    neg = dense_ops.linear(h, cand)                                                       # [T, C] bf16 on CUDA
    loss, hit = sampled_softmax.sampled_softmax_loss(pos, neg, cand_ids, target_ids, target_weights, self.temperature)
    return loss, hit.detach()
