"""Dense-gradient averaging across data-parallel ranks.

Two implementations behind one interface:
  * `FusedNvlinkReducer` (CUDA, one node): packs gradients into a symmetric-memory
    bucket in bf16, then ONE kernel performs a two-shot all-reduce over NVLink peer
    pointers with the 1/W scaling fused into the reduction (`csrc/cuda/allreduce.cu`).
  * `CollectiveReducer`: flat-bucket `dist.all_reduce` (gloo on CPU, NCCL as the
    stand-in baseline on GPU).
This replaces the all-reduce XLA inserts for replicated parameters in the reference
(`recml/core/training/partitioning.py:128-139`).
"""
from __future__ import annotations

import os
from typing import Sequence

import torch
import torch.distributed as dist


class CollectiveReducer:
  def __init__(self, group=None, bucket_bytes: int = 64 << 20):
    self.group = group
    self.bucket_bytes = bucket_bytes

  def average_grads(self, params: Sequence[torch.Tensor]) -> None:
    world = dist.get_world_size(self.group)
    bucket, size = [], 0
    for p in params:
      bucket.append(p)
      size += p.grad.numel() * p.grad.element_size()
      if size >= self.bucket_bytes:
        self._reduce(bucket, world)
        bucket, size = [], 0
    if bucket:
      self._reduce(bucket, world)

  def _reduce(self, bucket, world):
    flat = torch.cat([p.grad.reshape(-1).to(torch.float32) for p in bucket])
    dist.all_reduce(flat, group=self.group)
    flat.div_(world)
    off = 0
    for p in bucket:
      n = p.grad.numel()
      p.grad.copy_(flat[off:off + n].view_as(p.grad))
      off += n


def make_reducer(group, device: torch.device):
  if device.type == "cuda" and os.environ.get("RECML_COMM", "fused") == "fused":
    from recml_b200.comm import symm
    if symm.available(group):
      from recml_b200.comm import fused_allreduce
      return fused_allreduce.FusedNvlinkReducer(group, device)
  return CollectiveReducer(group)
