"""Thin wrappers over the memory-bound helper kernels (`csrc/cuda/elementwise.cu`).
Every function has a torch fallback for CPU tensors that doubles as the test oracle."""
from __future__ import annotations

import ctypes

import torch

from recml_b200.ops import _lib

c_ll, c_int, c_float = ctypes.c_longlong, ctypes.c_int, ctypes.c_float


def cast_bf16(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
  if not x.is_cuda:
    return x.to(torch.bfloat16)
  x = x.contiguous()
  out = torch.empty_like(x, dtype=torch.bfloat16) if out is None else out
  _lib.check_rc(_lib.cuda().recml_cast_f32_bf16(_lib.ptr(x), _lib.ptr(out), c_ll(x.numel()), _lib.stream()),
                "cast_f32_bf16")
  return out


def cast_pad_rows(x: torch.Tensor, cols_out: int, out: torch.Tensor | None = None) -> torch.Tensor:
  """fp32 `[M, C]` → bf16 `[M, cols_out]` zero-padded (TMA needs 16-byte row pitches)."""
  M, C = x.shape
  if not x.is_cuda:
    o = torch.zeros(M, cols_out, dtype=torch.bfloat16)
    o[:, :C] = x.to(torch.bfloat16)
    return o
  out = torch.empty(M, cols_out, dtype=torch.bfloat16, device=x.device) if out is None else out
  _lib.check_rc(_lib.cuda().recml_cast_pad_rows(_lib.ptr(x.contiguous()), c_int(C), _lib.ptr(out), c_int(cols_out),
                                                c_ll(out.stride(0)), c_ll(M), _lib.stream()), "cast_pad_rows")
  return out


def colsum(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
  """fp32 `[N]` column sums of a bf16 `[M, N]` matrix (row stride may exceed N)."""
  M, N = x.shape
  if not x.is_cuda:
    s = x.to(torch.float32).sum(0)
    return s if out is None else out.add_(s)
  if out is None:
    out = torch.zeros(N, dtype=torch.float32, device=x.device)
  _lib.check_rc(_lib.cuda().recml_colsum_bf16(_lib.ptr(x), c_ll(M), c_int(N), c_ll(x.stride(0)), _lib.ptr(out),
                                              _lib.stream()), "colsum")
  return out


def cross_bwd_ew(g, x0, v, dx0, accumulate: bool, want_colsum: bool = False):
  """dv = g⊙x0 (returned); dx0 (+)= g⊙v, in place.  With `want_colsum` also returns the fp32 column
  sums of dv (the cross layer's bias gradient), computed in the same pass."""
  if not g.is_cuda:
    dv = (g.float() * x0.float()).to(g.dtype)
    upd = g.float() * v.float()
    dx0.copy_((dx0.float() + upd if accumulate else upd).to(dx0.dtype))
    return (dv, dv.float().sum(0)) if want_colsum else dv
  M, N = g.shape
  assert g.stride(0) == x0.stride(0) == v.stride(0) == dx0.stride(0)
  dv = torch.empty_strided(g.shape, g.stride(), dtype=g.dtype, device=g.device)
  cs = torch.zeros(N, dtype=torch.float32, device=g.device) if want_colsum else None
  _lib.check_rc(_lib.cuda().recml_cross_bwd_ew(_lib.ptr(g), _lib.ptr(x0), _lib.ptr(v), _lib.ptr(dv), _lib.ptr(dx0),
                                               c_int(int(accumulate)), c_ll(M), c_int(N), c_ll(g.stride(0)),
                                               _lib.ptr(cs), _lib.stream()), "cross_bwd_ew")
  return (dv, cs) if want_colsum else dv


def add_bf16(a, b, out=None):
  if not a.is_cuda:
    return (a.float() + b.float()).to(a.dtype)
  M, N = a.shape
  out = torch.empty(M, N, dtype=a.dtype, device=a.device) if out is None else out
  _lib.check_rc(_lib.cuda().recml_add_bf16(_lib.ptr(a), c_ll(a.stride(0)), _lib.ptr(b), c_ll(b.stride(0)),
                                           _lib.ptr(out), c_ll(out.stride(0)), c_ll(M), c_int(N), _lib.stream()),
                "add_bf16")
  return out


def relu_mask(dy, y, out=None):
  if not dy.is_cuda:
    return torch.where(y > 0, dy, torch.zeros_like(dy))
  M, N = dy.shape
  out = torch.empty(M, N, dtype=dy.dtype, device=dy.device) if out is None else out
  _lib.check_rc(_lib.cuda().recml_relu_mask_bf16(_lib.ptr(dy), c_ll(dy.stride(0)), _lib.ptr(y), c_ll(y.stride(0)),
                                                 _lib.ptr(out), c_ll(out.stride(0)), c_ll(M), c_int(N),
                                                 _lib.stream()), "relu_mask")
  return out


def silu_bf16(z: torch.Tensor) -> torch.Tensor:
  """SiLU of a contiguous bf16 tensor (one pass, tanh-based)."""
  h = torch.empty_like(z)
  _lib.check_rc(_lib.cuda().recml_silu_fwd_bf16(_lib.ptr(z), _lib.ptr(h), c_ll(z.numel()), _lib.stream()), "silu_fwd")
  return h


def silu_split(z: torch.Tensor):
  """silu(z) for `z [T, 4 D]` as (u `[T, D]`, qkv `[T, 3 D]`), both contiguous."""
  T, W4 = z.shape
  D = W4 // 4
  u = torch.empty(T, D, dtype=z.dtype, device=z.device)
  qkv = torch.empty(T, 3 * D, dtype=z.dtype, device=z.device)
  _lib.check_rc(_lib.cuda().recml_silu_fwd_split(_lib.ptr(z), _lib.ptr(u), _lib.ptr(qkv), c_ll(T), c_int(D),
                                                 _lib.stream()), "silu_fwd_split")
  return u, qkv


def silu_bwd_gather4(z, g0, g1_f32, g2, g3):
  """dz `[T, 4 D]` = (g0 | g1 | g2 | g3) * silu'(z) for the pre-activation `z [T, 4 D]` of a fused four-way
  projection: g0 bf16 `[T, D]` (any row pitch), g1 fp32 `[T, D]`, g2 / g3 bf16 `[T, D]`, all with unit column
  stride."""
  T, W4 = z.shape
  D = W4 // 4
  dz = torch.empty_like(z)
  _lib.check_rc(_lib.cuda().recml_silu_bwd_gather4(_lib.ptr(z), _lib.ptr(g0), c_ll(g0.stride(0)), _lib.ptr(g1_f32),
                                                   _lib.ptr(g2), _lib.ptr(g3), _lib.ptr(dz), c_ll(T), c_int(D),
                                                   _lib.stream()), "silu_bwd_gather4")
  return dz


def gemv_fwd(x, w, bias):
  """fp32 `[M]` = bf16 `[M, K]` · fp32 `[K]` + bias."""
  if not x.is_cuda:
    return x.float() @ w.float() + (bias.float() if bias is not None else 0.0)
  M, K = x.shape
  y = torch.empty(M, dtype=torch.float32, device=x.device)
  _lib.check_rc(_lib.cuda().recml_gemv_fwd(_lib.ptr(x), c_ll(x.stride(0)), c_int(K), _lib.ptr(w), _lib.ptr(bias),
                                           _lib.ptr(y), c_ll(M), _lib.stream()), "gemv_fwd")
  return y


def gemv_bwd(x, w, dy, mask_relu: bool, dw, db):
  """Returns dx bf16 `[M, K]`; accumulates into fp32 `dw [K]`, `db [1]`."""
  if not x.is_cuda:
    dx = dy[:, None].float() * w[None, :].float()
    if mask_relu:
      dx = torch.where(x > 0, dx, torch.zeros_like(dx))
    dw += (dy[:, None].float() * x.float()).sum(0)
    if db is not None:
      db += dy.sum()
    return dx.to(x.dtype)
  M, K = x.shape
  dx = torch.empty(M, K, dtype=torch.bfloat16, device=x.device)
  _lib.check_rc(_lib.cuda().recml_gemv_bwd(_lib.ptr(x), c_ll(x.stride(0)), c_int(K), _lib.ptr(w), _lib.ptr(dy),
                                           c_ll(M), _lib.ptr(dx), c_ll(dx.stride(0)), c_int(int(mask_relu)),
                                           _lib.ptr(dw), _lib.ptr(db), _lib.stream()), "gemv_bwd")
  return dx
