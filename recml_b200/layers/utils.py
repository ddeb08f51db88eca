"""Layer helpers (`recml/layers/keras/utils.py:22-147`): attention masks, activations, the L2
embedding post-processor, rotary encodings."""
from __future__ import annotations

import copy
from typing import Any

import torch


def clone_initializer(initializer: Any) -> Any:
  return copy.deepcopy(initializer)


def make_attention_mask(mask: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
  """`[B, L]` padding mask → `[B, L, L]` pairwise mask."""
  return (mask.unsqueeze(-1) * mask.unsqueeze(-2)).to(dtype)


def make_causal_mask(mask: torch.Tensor, dtype: torch.dtype = torch.float32) -> torch.Tensor:
  return torch.tril(make_attention_mask(mask, dtype))


def gelu_approximate(x: torch.Tensor) -> torch.Tensor:
  return torch.nn.functional.gelu(x, approximate="tanh")


def relu_squared(x: torch.Tensor) -> torch.Tensor:
  return torch.relu(x) ** 2


def norm_embedding_post_processor(inputs: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
  """Scales every embedding to unit L2 norm (norm clipped below at eps)."""
  return inputs / inputs.norm(dim=-1, keepdim=True).clamp_min(eps)


def apply_rotary_encoding(x: torch.Tensor, *, positions: torch.Tensor | None = None,
                          max_wavelength: int) -> torch.Tensor:
  """RoPE on `[*batch, L, H, Dh]` (Dh even): halves are rotated by position/timescale."""
  if x.shape[-1] % 2:
    raise ValueError(f"Embedding dimension must be even, but got {x.shape[-1]} for input of shape {tuple(x.shape)}.")
  if x.ndim < 4:
    raise ValueError(f"Unexpected input shape: {tuple(x.shape)}. Expected shape of rank 4 or greater.")
  L, half = x.shape[-3], x.shape[-1] // 2
  if positions is None:
    positions = torch.arange(L, device=x.device).expand(*x.shape[:-3], L)
  elif tuple(positions.shape) != tuple(x.shape[:-2]):
    raise ValueError(f"Positions must be of shape: {tuple(x.shape[:-2])} but got shape: {tuple(positions.shape)}.")
  exponents = (2.0 / x.shape[-1]) * torch.arange(half, dtype=torch.float32, device=x.device)
  timescale = float(max_wavelength) ** exponents
  radians = positions.to(torch.float32)[..., None] / timescale          # [..., L, half]
  radians = radians[..., None, :]                                        # [..., L, 1, half]
  sin, cos = torch.sin(radians), torch.cos(radians)
  x1, x2 = x[..., :half].float(), x[..., half:].float()
  return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


def large_negative_for_attention(dtype: torch.dtype) -> float:
  return -3e4 if dtype == torch.float16 else -1e9
