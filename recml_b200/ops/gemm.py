"""bf16 tensor-core GEMM (`csrc/cuda/gemm_tcgen05.cu`) and its torch reference.

`gemm(a, b, ...)` computes `epilogue(A·Bᵀ)` where A is logically `[M, K]` and B logically
`[N, K]`; `a_mn` / `b_mn` say that the tensor handed in is the TRANSPOSE of that logical
operand (stored `[K, M]` / `[K, N]`), which is how backward passes avoid transposes.
On CPU tensors the same contract is evaluated with torch in fp32 (the test oracle).
"""
from __future__ import annotations

import ctypes

import torch

from recml_b200.ops import _lib

EPI_LINEAR, EPI_CROSS, EPI_MASK_RELU, EPI_MUL_ADD, EPI_ADD = 0, 1, 2, 3, 4


def gemm_reference(a, b, *, a_mn=False, b_mn=False, bias=None, relu=False, epi=EPI_LINEAR,
                   aux0=None, aux1=None, out_dtype=torch.bfloat16, accumulate_into=None,
                   want_out2=False):
  A = a.to(torch.float32).t() if a_mn else a.to(torch.float32)
  B = b.to(torch.float32).t() if b_mn else b.to(torch.float32)
  x = A @ B.t()
  if bias is not None:
    x = x + bias.to(torch.float32)
  out2 = None
  if epi == EPI_LINEAR:
    if relu:
      x = torch.relu(x)
  elif epi == EPI_CROSS:
    out2 = x.to(torch.bfloat16) if want_out2 else None
    x = aux0.to(torch.float32) * x + aux1.to(torch.float32)
  elif epi == EPI_MASK_RELU:
    x = torch.where(aux0 > 0, x, torch.zeros_like(x))
  elif epi == EPI_ADD:
    x = x + aux0.to(torch.float32)
    if aux1 is not None:
      x = x + aux1.to(torch.float32)
  elif epi == EPI_MUL_ADD:
    x = x * aux0.to(torch.float32)
    if aux1 is not None:
      x = x + aux1.to(torch.float32)
  if accumulate_into is not None:
    accumulate_into += x
    return (accumulate_into, out2) if want_out2 else accumulate_into
  x = x.to(out_dtype)
  return (x, out2) if want_out2 else x


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: torch.Tensor | None = None, relu: bool = False, epi: int = EPI_LINEAR,
         aux0: torch.Tensor | None = None, aux1: torch.Tensor | None = None,
         out_dtype: torch.dtype = torch.bfloat16, out: torch.Tensor | None = None,
         accumulate_into: torch.Tensor | None = None, want_out2: bool = False, split_k: int = 0):
  """`split_k=0` picks a K split automatically for fp32-output products whose tile count would
  leave most SMs idle (weight gradients: few output tiles, very long K)."""
  if not a.is_cuda:
    return gemm_reference(a, b, a_mn=a_mn, b_mn=b_mn, bias=bias, relu=relu, epi=epi, aux0=aux0,
                          aux1=aux1, out_dtype=out_dtype, accumulate_into=accumulate_into,
                          want_out2=want_out2)
  assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "operands must be bf16"
  assert a.stride(-1) == 1 and b.stride(-1) == 1
  K, M = (a.shape if a_mn else a.shape[::-1])
  Kb, N = (b.shape if b_mn else b.shape[::-1])
  assert K == Kb, f"contraction mismatch {a.shape} {b.shape} a_mn={a_mn} b_mn={b_mn}"
  if accumulate_into is not None:
    d, out_f32, acc = accumulate_into, 1, 1
    assert d.dtype == torch.float32
  else:
    d = out if out is not None else _lib.debug_empty((M, N), out_dtype, a.device, f"gemm output [{M}, {N}]")
    out_f32, acc = int(d.dtype == torch.float32), 0
  out2 = _lib.debug_empty((M, N), torch.bfloat16, a.device, "gemm second output") if want_out2 else None
  if split_k == 0:
    split_k = 1
    if out_f32 and epi == EPI_LINEAR and bias is None and not relu:
      tiles = ((M + 127) // 128) * ((N + 255) // 256 if N > 128 else 1)
      kb = (K + 63) // 64
      if tiles < 148 and kb >= 32:
        split_k = max(1, min(296 // tiles, kb // 16, 16))
  if split_k > 1 and not acc:
    d.zero_()
  ldaux = aux0.stride(0) if aux0 is not None else 0
  rc = _lib.cuda().recml_gemm_bf16(
      _lib.ptr(a), ctypes.c_int(a.stride(0)), ctypes.c_int(int(a_mn)),
      _lib.ptr(b), ctypes.c_int(b.stride(0)), ctypes.c_int(int(b_mn)),
      _lib.ptr(d), ctypes.c_int(d.stride(0)), ctypes.c_int(out_f32), ctypes.c_int(acc),
      ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), _lib.ptr(bias), ctypes.c_int(int(relu)),
      ctypes.c_int(epi), _lib.ptr(aux0), _lib.ptr(aux1), ctypes.c_int(ldaux), _lib.ptr(out2),
      ctypes.c_int(split_k), _lib.ptr(_lib.status_buffer(a.device)), _lib.stream())
  _lib.check_rc(rc, "recml_gemm_bf16")
  return (d, out2) if want_out2 else d
