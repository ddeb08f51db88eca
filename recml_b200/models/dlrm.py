"""DLRM-DCNv2: bottom MLP on dense features, sharded embedding bags, DCNv2 cross network, top MLP.

Same model as the reference's (`recml/examples/dlrm_experiment.py:98-194`,
`recml/inference/models/jax/DLRM_DCNv2/dlrm_model.py:42-168`): concat order is
`[bottom_out, *sparse features]`, the cross network runs on the concat and the top MLP ends in
one logit (no sigmoid; the loss is BCE-with-logits).  On CUDA every matrix product runs on the
tcgen05 GEMM and the embedding bags on the fused sharded-embedding kernels.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from recml_b200 import embedding as emb
from recml_b200.layers import dcn, dense


class DLRMDCNv2(nn.Module):
  def __init__(self, *, vocab_sizes: Sequence[int], embedding_dim: int = 128, num_dense: int = 13,
               bottom_mlp_dims: Sequence[int] = (512, 256, 128),
               top_mlp_dims: Sequence[int] = (1024, 1024, 512, 256, 1), num_cross_layers: int = 3,
               cross_rank: int | None = 512, bag_sizes: Sequence[int] | None = None,
               embedding_optimizer: emb.OptimizerSpec | None = None, combiner: str = "sum",
               feature_names: Sequence[str] | None = None, device=None, group=None,
               sharding_strategy: str = "auto", row_wise_min_bytes: int | None = None,
               backend: str = "auto", seed: int = 0, init_scale: float | None = None,
               overlap_backward: bool = True, hot_row_share: Sequence | None = None,
               residue_stats=None, allow_id_dropping: bool = False):
    super().__init__()
    if bottom_mlp_dims[-1] != embedding_dim:
      raise ValueError("bottom MLP must end in embedding_dim so it can join the feature concat")
    names = list(feature_names) if feature_names else [f"cat_{i}" for i in range(len(vocab_sizes))]
    self.feature_names = names
    init = (lambda v: emb.specs.uniform_init((1.0 / v) ** 0.5)) if init_scale is None else \
        (lambda v: emb.specs.normal_init(init_scale))
    specs = {n: emb.EmbeddingSpec(input_dim=v, embedding_dim=embedding_dim, combiner=combiner,
                                  initializer=init(v)) for n, v in zip(names, vocab_sizes)}
    ids = {n: float(b) for n, b in zip(names, bag_sizes)} if bag_sizes is not None else None
    self.embedding = emb.ShardedEmbedding(
        emb.ShardedEmbeddingConfig(
            specs, embedding_optimizer or emb.RowWiseAdagradOptimizerSpec(learning_rate=0.01),
            sharding_strategy=sharding_strategy, row_wise_min_bytes=row_wise_min_bytes,
            ids_per_sample=ids, backend=backend, seed=seed, allow_id_dropping=allow_id_dropping,
            # share of each feature's ids on its most frequent row: lets the planner offset the rank that holds the
            # hot row of a row-sharded table
            hot_row_share=dict(zip(names, hot_row_share)) if hot_row_share is not None else None,
            # ids and distinct ids per residue class, measured on a batch (see `embedding.stats`)
            residue_stats=residue_stats),
        device=device, group=group)
    self.bottom = dense.MLP([num_dense, *bottom_mlp_dims], activate_last=True)
    d = embedding_dim * (1 + len(vocab_sizes))
    self.cross = dcn.CrossNetwork(d, num_cross_layers, cross_rank)
    self.top = dense.MLP([d, *top_mlp_dims], activate_last=False)
    self.concat_dim = d
    if device is not None:
      self.bottom.to(device); self.cross.to(device); self.top.to(device)
    # Backward schedule on CUDA: the data-gradient chain of the top MLP and the cross network runs first;
    # its end feeds the embedding backward (its own stream, memory-latency bound), beside which the queued
    # weight-gradient GEMMs (tensor-core bound) run on a third stream.
    if overlap_backward and device is not None and torch.device(device).type == "cuda":
      self.cross.defer_wgrad = True
      self.top.defer_wgrad = True
      backend_obj = getattr(self.embedding, "_backend", None)
      if hasattr(backend_obj, "bwd_blocks_per_sm") and backend_obj.bwd_blocks_per_sm == 0:
        backend_obj.bwd_blocks_per_sm = -1

  def forward(self, dense_x: torch.Tensor, sparse: emb.KeyedJagged) -> torch.Tensor:
    if dense_x.is_cuda:
      # bottom MLP and embedding kernels write their halves of the concat in place
      from recml_b200.ops import dense as dense_ops
      k = self.bottom.dims[-1]
      full = torch.empty(dense_x.shape[0], self.concat_dim, dtype=torch.bfloat16, device=dense_x.device)
      bottom = self.bottom(dense_x, out=full[:, :k])
      pooled = self.embedding(sparse, flat=True, out=full, out_col=k)
      x0 = dense_ops.JoinColumnsFn.apply(bottom, pooled, full)
    else:
      bottom = self.bottom(dense_x)
      pooled = self.embedding(sparse, flat=True)
      x0 = torch.cat([bottom.to(pooled.dtype), pooled], dim=1)
    y = self.top(self.cross(x0))
    return y.reshape(-1).to(torch.float32)
