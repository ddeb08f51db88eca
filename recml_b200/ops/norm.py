"""LayerNorm family (`csrc/cuda/layernorm.cu` on CUDA, torch on CPU): standard LN over the last
dim, LN over the last two dims jointly (HSTU attention output, `recml/layers/keras/hstu.py:340-343`),
with the `u ⊙ LN(x)` gate fused, and the RMS-scaled gated norm of Mamba2
(`recml/layers/keras/mamba.py:257-263,413`)."""
from __future__ import annotations

import ctypes

import torch

from recml_b200.ops import _lib


def _ln_ref(x, w, b, eps, rms=False):
  xf = x.float()
  if rms:
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
  else:
    mu = xf.mean(-1, keepdim=True)
    y = (xf - mu) * torch.rsqrt(xf.var(-1, unbiased=False, keepdim=True) + eps)
  if w is not None:
    y = y * w.float()
  if b is not None:
    y = y + b.float()
  return y


class _LayerNormFn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, x, w, b, gate, eps, rms):
    D = w.numel()
    x2 = x.detach().reshape(-1, D).contiguous()
    g2 = None if gate is None else gate.detach().reshape(-1, D).contiguous()
    M = x2.shape[0]
    y = torch.empty_like(x2)
    stats = torch.empty(M, 2, dtype=torch.float32, device=x.device)
    rc = _lib.cuda().recml_layernorm_fwd(
        _lib.ptr(x2), _lib.ptr(g2), _lib.ptr(w.detach().float().contiguous()),
        _lib.ptr(None if b is None else b.detach().float().contiguous()), _lib.ptr(y), _lib.ptr(stats),
        ctypes.c_longlong(M), ctypes.c_int(D), ctypes.c_float(eps), ctypes.c_int(int(rms)),
        ctypes.c_int(int(x2.dtype == torch.bfloat16)), _lib.stream())
    _lib.check_rc(rc, "layernorm_fwd")
    ctx.save_for_backward(x2, g2, w, stats)
    ctx.bias = None if b is None else b.detach().float().contiguous()
    ctx.meta = (x.shape, D, rms, b is not None, gate is not None)
    return y.view(x.shape)

  @staticmethod
  def backward(ctx, dy):
    x2, g2, w, stats = ctx.saved_tensors
    shape, D, rms, has_b, has_gate = ctx.meta
    dy2 = dy.reshape(-1, D).contiguous().to(x2.dtype)
    M = x2.shape[0]
    dx = torch.empty_like(x2)
    dgate = torch.empty_like(x2) if has_gate else None
    dw = torch.zeros(D, dtype=torch.float32, device=x2.device)
    db = torch.zeros(D, dtype=torch.float32, device=x2.device)
    rc = _lib.cuda().recml_layernorm_bwd(
        _lib.ptr(dy2), _lib.ptr(x2), _lib.ptr(g2), _lib.ptr(w.detach().float().contiguous()), _lib.ptr(ctx.bias),
        _lib.ptr(stats),
        _lib.ptr(dx), _lib.ptr(dgate), _lib.ptr(dw), _lib.ptr(db), ctypes.c_longlong(M), ctypes.c_int(D),
        ctypes.c_int(int(rms)), ctypes.c_int(int(x2.dtype == torch.bfloat16)), _lib.stream())
    _lib.check_rc(rc, "layernorm_bwd")
    return (dx.view(shape), dw.to(w.dtype).view_as(w), db.to(w.dtype).view_as(w) if has_b else None,
            dgate.view(shape) if has_gate else None, None, None)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float = 1e-6, *,
               gate: torch.Tensor | None = None, rms: bool = False, norm_dims: int = 1) -> torch.Tensor:
  """y = gate ⊙ (LN(x)·w + b).  `norm_dims=2` normalises over the last two dims jointly (weight has
  that shape).  `rms=True` drops the mean subtraction (Keras `rms_scaling`)."""
  if norm_dims == 2:
    shp = x.shape
    x = x.reshape(*shp[:-2], shp[-2] * shp[-1])
    gate = None if gate is None else gate.reshape(x.shape)
    y = layer_norm(x, weight.reshape(-1), None if bias is None else bias.reshape(-1), eps, gate=gate, rms=rms)
    return y.view(shp)
  D = x.shape[-1]
  if not x.is_cuda or D > 1024 or x.dtype not in (torch.bfloat16, torch.float32):
    y = _ln_ref(x, weight, bias, eps, rms)
    if gate is not None:
      y = y * gate.float()
    return y.to(x.dtype)
  return _LayerNormFn.apply(x, weight, bias, gate, eps, rms)
