"""Dense layers: `Linear`, `MLP` (DLRM bottom / top towers, `recml/examples/
dlrm_experiment.py:136-152`).  Parameters are fp32 masters in the torch `[out, in]` layout; CUDA
execution uses bf16 copies on the tcgen05 GEMM (`recml_b200.ops.dense`)."""
from __future__ import annotations

import math
from typing import Sequence

import torch
from torch import nn

from recml_b200.ops import dense as dense_ops


def lecun_normal_(w: torch.Tensor) -> None:
  fan_in = w.shape[1]
  std = math.sqrt(1.0 / fan_in) / 0.87962566103423978  # truncated-normal variance correction
  nn.init.trunc_normal_(w, 0.0, std, -2 * std, 2 * std)


class Linear(nn.Module):
  def __init__(self, in_features: int, out_features: int, bias: bool = True, activation: str | None = None,
               init=lecun_normal_):
    super().__init__()
    self.weight = nn.Parameter(torch.empty(out_features, in_features))
    self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
    self.activation = activation
    init(self.weight)

  def forward(self, x):
    if self.activation in (None, "relu"):
      return dense_ops.linear(x, self.weight, self.bias, relu=self.activation == "relu")
    y = dense_ops.linear(x, self.weight, self.bias)
    return getattr(torch.nn.functional, self.activation)(y)


class MLP(nn.Module):
  """`dims = [in, h1, ..., out]`; ReLU after every layer except the last unless
  `activate_last`."""

  def __init__(self, dims: Sequence[int], activate_last: bool = False, bias: bool = True):
    super().__init__()
    self.dims = list(dims)
    self.weights = nn.ParameterList()
    self.biases = nn.ParameterList() if bias else None
    for i in range(len(dims) - 1):
      w = torch.empty(dims[i + 1], dims[i])
      lecun_normal_(w)
      self.weights.append(nn.Parameter(w))
      if bias:
        self.biases.append(nn.Parameter(torch.zeros(dims[i + 1])))
    n = len(dims) - 1
    self.relu_flags = [True] * (n - 1) + [bool(activate_last)]
    # set by a model that flushes `ops.dense` deferred weight gradients itself (see `ops/dense.py`)
    self.defer_wgrad = False

  def forward(self, x, out=None):
    biases = list(self.biases) if self.biases is not None else [None] * len(self.weights)
    return dense_ops.mlp(x, list(self.weights), biases, self.relu_flags, out=out,
                         defer_wgrad=self.defer_wgrad and x.is_cuda and torch.is_grad_enabled())
