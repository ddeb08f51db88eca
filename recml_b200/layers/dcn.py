"""DCNv2 cross network (`recml/examples/dlrm_experiment.py:154-177`): low-rank
`xl ← x0 ⊙ ((xl·U)·V + b) + xl` with xavier-normal kernels and zero bias, plus the full-rank
variant `xl ← x0 ⊙ (W·xl + b) + xl`."""
from __future__ import annotations

import torch
from torch import nn

from recml_b200.ops import dense as dense_ops


class CrossNetwork(nn.Module):
  def __init__(self, dim: int, num_layers: int, rank: int | None = None):
    super().__init__()
    self.dim, self.num_layers, self.rank = dim, num_layers, rank
    self.u = nn.ParameterList() if rank else None
    self.v = nn.ParameterList()
    self.b = nn.ParameterList()
    for _ in range(num_layers):
      if rank:
        u = torch.empty(rank, dim)      # applied as xl·Uᵀ  (the reference's u_kernel [d, r], transposed)
        v = torch.empty(dim, rank)
        nn.init.xavier_normal_(u)
        nn.init.xavier_normal_(v)
        self.u.append(nn.Parameter(u))
      else:
        v = torch.empty(dim, dim)
        nn.init.xavier_normal_(v)
      self.v.append(nn.Parameter(v))
      self.b.append(nn.Parameter(torch.zeros(dim)))
    self.defer_wgrad = False   # see `MLP.defer_wgrad`

  def forward(self, x0):
    return dense_ops.cross_network(x0, list(self.u) if self.u is not None else None, list(self.v), list(self.b),
                                   defer_wgrad=self.defer_wgrad and x0.is_cuda and torch.is_grad_enabled())
