"""State-space duality (SSD) scan of Mamba2 and the depthwise causal conv that precedes it.

  h_t = exp(a_t)·h_{t−1} + b_t ⊗ x_t ,   y_t = c_t · h_t          (per head; b, c shared in a group)

Computed chunk-wise like the reference (`recml/layers/keras/mamba.py:53-146`): inside a chunk the
output is a masked "attention" (C·Bᵀ ⊙ decay)·X, chunk end-states are carried by a short
sequential recurrence, and the carried state contributes C·state·decay.  `ssd_recurrent` is the
plain O(L) recurrence used as the oracle.  On CUDA the chunk kernels are `csrc/cuda/ssd.cu`.
"""
from __future__ import annotations

import torch


def ssd_recurrent(x, a, b, c, initial_state=None):
  """x `[B, L, H, P]`, a `[B, L, H]`, b / c `[B, L, G, N]` → y `[B, L, H, P]` (fp32 recurrence)."""
  B, L, H, P = x.shape
  G, N = b.shape[-2:]
  rep = H // G
  h = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device) if initial_state is None \
      else initial_state.float().clone()
  ys = []
  bf, cf = b.float().repeat_interleave(rep, dim=2), c.float().repeat_interleave(rep, dim=2)
  for t in range(L):
    h = h * torch.exp(a[:, t].float())[..., None, None] + x[:, t].float()[..., None] * bf[:, t][:, :, None, :]
    ys.append(torch.einsum("bhpn,bhn->bhp", h, cf[:, t]))
  return torch.stack(ys, dim=1).to(x.dtype)


def ssd_chunked(x, a, b, c, block_len: int, initial_states=None):
  """Same contract as the reference's `ssd_minimal_discrete` (L must be a multiple of block_len)."""
  B, L, H, P = x.shape
  G, N = b.shape[-2:]
  assert L % block_len == 0, "sequence length must be a multiple of the chunk size"
  assert G == 1 or G == H, "groups must be 1 or equal to heads"
  C = L // block_len
  xf = x.float().reshape(B, C, block_len, H, P)
  af = a.float().reshape(B, C, block_len, H).permute(0, 3, 1, 2)           # [B, H, C, l]
  bf = b.float().reshape(B, C, block_len, G, N).expand(B, C, block_len, H, N) if G == 1 else \
      b.float().reshape(B, C, block_len, H, N)
  cf = c.float().reshape(B, C, block_len, G, N).expand(B, C, block_len, H, N) if G == 1 else \
      c.float().reshape(B, C, block_len, H, N)
  cum = torch.cumsum(af, dim=-1)                                            # inclusive prefix of a
  # intra-chunk: decay[l, s] = exp(cum[l] − cum[s]) for s ≤ l
  diff = cum[..., :, None] - cum[..., None, :]
  tri = torch.tril(torch.ones(block_len, block_len, dtype=torch.bool, device=x.device))
  decay = torch.where(tri, torch.exp(diff.masked_fill(~tri, 0.0)), torch.zeros((), device=x.device))
  scores = torch.einsum("bclhn,bcshn->bhcls", cf, bf) * decay
  y_diag = torch.einsum("bhcls,bcshp->bclhp", scores, xf)
  # chunk end states
  to_end = torch.exp(cum[..., -1:] - cum)                                   # [B, H, C, l]
  states = torch.einsum("bclhn,bhcl,bclhp->bchpn", bf, to_end, xf)
  # carry across chunks (sequential over C, tiny)
  carry = torch.zeros(B, H, P, N, dtype=torch.float32, device=x.device) if initial_states is None \
      else initial_states.float().reshape(B, H, P, N)
  chunk_decay = torch.exp(cum[..., -1])                                     # [B, H, C]
  prev = []
  for ci in range(C):
    prev.append(carry)
    carry = carry * chunk_decay[:, :, ci][..., None, None] + states[:, ci]
  prev = torch.stack(prev, dim=1)                                           # state entering each chunk
  y_off = torch.einsum("bclhn,bchpn,bhcl->bclhp", cf, prev, torch.exp(cum))
  return (y_diag + y_off).reshape(B, L, H, P).to(x.dtype)


def causal_depthwise_conv1d_silu(x, weight, bias=None):
  """x `[B, L, C]`, weight `[C, K]` (tap k multiplies x[t − (K−1) + k]); SiLU fused."""
  K = weight.shape[1]
  xp = torch.nn.functional.pad(x.float().transpose(1, 2), (K - 1, 0))
  y = torch.nn.functional.conv1d(xp, weight.float()[:, None, :], None if bias is None else bias.float(),
                                 groups=weight.shape[0])
  return torch.nn.functional.silu(y).transpose(1, 2).to(x.dtype)
