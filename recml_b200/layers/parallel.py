"""Tensor-parallel linear layers (Megatron-style column / row split) over one mesh axis.

The reference gets tensor parallelism from the compiler: a kernel annotated with
`nn.with_partitioning(..., (None, "model"))` makes GSPMD split the matmul and insert the collectives
(`recml/core/training/partitioning.py:148-288`).  Here the split is a property of the layer:

  ColumnParallelLinear   W `[out, in]` is cut along `out`: every rank computes its slice of the output from
                         the whole input; backward all-reduces the input gradient.  `gather_output=True`
                         concatenates the slices (all-gather), else the next layer takes the slice as is.
  RowParallelLinear      W is cut along `in`: every rank multiplies its slice of the input (`input_is_split`)
                         and the partial products are summed (all-reduce); the bias is added once, after.

A column layer followed by a row layer needs one all-reduce forward and one backward, as usual.  The
layers hold only their own shards; `ModelParallelPartitioner` reads `_recml_tp_spec` from the parameters
to place them in checkpoints and to keep them out of the model-axis gradient reduction.  Collectives go
through `torch.distributed` (NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from recml_b200.layers import dense as dense_layers


def _size(group) -> int:
  return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def _rank(group) -> int:
  return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


class _CopyIn(torch.autograd.Function):
  """Identity forward; backward sums the gradient over the group (the input is replicated)."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    return x

  @staticmethod
  def backward(ctx, g):
    if _size(ctx.group) > 1:
      g = g.contiguous()
      dist.all_reduce(g, group=ctx.group)
    return g, None


class _ReduceOut(torch.autograd.Function):
  """Sums partial results over the group; backward is the identity."""

  @staticmethod
  def forward(ctx, x, group):
    if _size(group) > 1:
      x = x.contiguous().clone()
      dist.all_reduce(x, group=group)
    return x

  @staticmethod
  def backward(ctx, g):
    return g, None


class _GatherLast(torch.autograd.Function):
  """Concatenates the ranks' slices along the last dim; backward keeps the own slice."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    n = _size(group)
    if n == 1:
      return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=-1)

  @staticmethod
  def backward(ctx, g):
    n = _size(ctx.group)
    if n == 1:
      return g, None
    return g.chunk(n, dim=-1)[_rank(ctx.group)].contiguous(), None


class _SplitLast(torch.autograd.Function):
  """Keeps the own slice of the last dim; backward concatenates the ranks' gradients."""

  @staticmethod
  def forward(ctx, x, group):
    ctx.group = group
    n = _size(group)
    return x if n == 1 else x.chunk(n, dim=-1)[_rank(group)].contiguous()

  @staticmethod
  def backward(ctx, g):
    n = _size(ctx.group)
    if n == 1:
      return g, None
    parts = [torch.empty_like(g) for _ in range(n)]
    dist.all_gather(parts, g.contiguous(), group=ctx.group)
    return torch.cat(parts, dim=-1), None


def _init_full(out_features: int, in_features: int, seed: int) -> torch.Tensor:
  """The full weight, generated identically on every rank, so that a split layer starts from the same
  values as the dense layer it replaces (whatever the number of ranks)."""
  gen = torch.Generator().manual_seed(seed)
  std = math.sqrt(1.0 / in_features)
  return torch.randn(out_features, in_features, generator=gen) * std


class ColumnParallelLinear(nn.Module):
  def __init__(self, in_features: int, out_features: int, *, group=None, axis: str = "model", bias: bool = True,
               gather_output: bool = False, activation: str | None = None, seed: int = 0):
    super().__init__()
    n, r = _size(group), _rank(group)
    if out_features % n:
      raise ValueError(f"out_features {out_features} not divisible by {n} ranks")
    self.group, self.gather_output, self.activation = group, gather_output, activation
    full = _init_full(out_features, in_features, seed)
    self.weight = nn.Parameter(full.chunk(n, dim=0)[r].clone())
    self.weight._recml_tp_spec = (axis, None)
    self.bias = None
    if bias:
      self.bias = nn.Parameter(torch.zeros(out_features // n))
      self.bias._recml_tp_spec = (axis,)

  def forward(self, x):
    x = _CopyIn.apply(x, self.group)
    y = dense_layers.dense_ops.linear(x, self.weight, self.bias, relu=self.activation == "relu")
    return _GatherLast.apply(y, self.group) if self.gather_output else y


class RowParallelLinear(nn.Module):
  def __init__(self, in_features: int, out_features: int, *, group=None, axis: str = "model", bias: bool = True,
               input_is_split: bool = True, seed: int = 1):
    super().__init__()
    n, r = _size(group), _rank(group)
    if in_features % n:
      raise ValueError(f"in_features {in_features} not divisible by {n} ranks")
    self.group, self.input_is_split = group, input_is_split
    full = _init_full(out_features, in_features, seed)
    self.weight = nn.Parameter(full.chunk(n, dim=1)[r].clone())
    self.weight._recml_tp_spec = (None, axis)
    self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None     # replicated, added after the sum

  def forward(self, x):
    if not self.input_is_split:
      x = _SplitLast.apply(x, self.group)
    y = _ReduceOut.apply(dense_layers.dense_ops.linear(x, self.weight, None), self.group)
    return y if self.bias is None else y + self.bias.to(y.dtype)


class TensorParallelMLP(nn.Module):
  """`in → hidden → out` with the hidden dim split over the group: column-parallel + ReLU, then
  row-parallel (one all-reduce per direction)."""

  def __init__(self, in_features: int, hidden: int, out_features: int, *, group=None, axis: str = "model",
               seed: int = 0):
    super().__init__()
    self.up = ColumnParallelLinear(in_features, hidden, group=group, axis=axis, activation="relu", seed=seed)
    self.down = RowParallelLinear(hidden, out_features, group=group, axis=axis, seed=seed + 1)

  def forward(self, x):
    return self.down(self.up(x))
