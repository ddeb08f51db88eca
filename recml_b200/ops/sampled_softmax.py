"""Sampled-softmax loss over one positive and C shared candidate logits per row.

The reference trains its sequence models with a full-vocabulary softmax
(`recml/examples/train_hstu_jax.py:160-163,177-180`); with a 10 M item table that is replaced by a
sampled softmax whose candidates are shared by all rows (uniform + in-batch negatives).  On CUDA the
loss, the hit-rate statistic and the gradient of the mean loss w.r.t. the logits come out of ONE kernel
(`csrc/cuda/sampled_softmax.cu`) that reads the bf16 candidate logits produced by the GEMM once and writes
the gradient once; the `[T, 1 + C]` fp32 logits, mask and probabilities are never materialised, and the
backward pass touches the gradient again only when the incoming loss gradient is not 1.
"""
from __future__ import annotations

import ctypes

import torch


def reference(pos, neg, cand_ids, target_ids, weights, temperature: float):
  """Plain torch formulation (also the CPU path): returns (mean loss, hit@1 among the candidates)."""
  neg = neg.float().masked_fill(cand_ids[None, :] == target_ids[:, None], -1e4)
  logits = torch.cat([pos.float().reshape(-1, 1), neg], dim=1) / temperature
  nll = torch.logsumexp(logits, dim=1) - logits[:, 0]
  w = weights.float()
  den = w.sum().clamp_min(1.0)
  loss = (nll * w).sum() / den
  hit = ((logits.argmax(dim=1) == 0).float() * w).sum() / den
  return loss, hit.detach()


class _Fn(torch.autograd.Function):
  @staticmethod
  def forward(ctx, pos, neg, cand_ids, target_ids, weights, temperature):
    from recml_b200.ops import _lib
    T, C = neg.shape
    posf = pos.float().reshape(-1).contiguous()
    negb = neg.to(torch.bfloat16)
    if negb.stride(1) != 1:
      negb = negb.contiguous()
    stats = torch.zeros(4, dtype=torch.float32, device=neg.device)
    dpos = torch.empty(T, dtype=torch.float32, device=neg.device)
    dneg = torch.empty_strided((T, C), (negb.stride(0), 1), dtype=torch.bfloat16, device=neg.device)
    w = weights.float().contiguous()
    den = w.sum().clamp_min(1.0).reshape(1)          # the kernel writes the gradient of the MEAN loss
    _lib.check_rc(_lib.cuda().recml_sampled_softmax(
        _lib.ptr(posf), _lib.ptr(negb), ctypes.c_longlong(negb.stride(0)), _lib.ptr(cand_ids.to(torch.int64).contiguous()),
        _lib.ptr(target_ids.to(torch.int64).contiguous()), _lib.ptr(w), ctypes.c_int(T), ctypes.c_int(C),
        ctypes.c_float(1.0 / temperature), _lib.ptr(den), _lib.ptr(stats), _lib.ptr(dpos), _lib.ptr(dneg), _lib.stream()),
        "sampled_softmax")
    ctx.save_for_backward(dpos, dneg)
    ctx.meta = (pos.dtype, pos.shape, neg.dtype)
    ctx.used = False
    ctx.mark_non_differentiable(hit := stats[2] / den[0])
    return stats[0] / den[0], hit

  @staticmethod
  def backward(ctx, g_loss, _g_hit):
    from recml_b200.ops import _lib
    if ctx.used:
      raise RuntimeError("the sampled-softmax gradient is scaled in place and can be propagated once")
    ctx.used = True
    dpos, dneg = ctx.saved_tensors
    pdt, pshape, ndt = ctx.meta
    g = g_loss.float().reshape(1).contiguous()
    # dneg *= g in place; a kernel that returns at once when g is exactly 1 (the plain `loss.backward()`), so the
    # usual step pays no extra pass over the [T, C] gradient
    T, C = dneg.shape
    _lib.check_rc(_lib.cuda().recml_scale_rows_bf16(_lib.ptr(dneg), ctypes.c_longlong(dneg.stride(0)), ctypes.c_int(T),
                                                    ctypes.c_int(C), _lib.ptr(g), _lib.stream()), "scale_rows")
    return (dpos * g).reshape(pshape).to(pdt), dneg.to(ndt), None, None, None, None


def sampled_softmax_loss(pos, neg, cand_ids, target_ids, weights, temperature: float):
  """pos `[T]` (or `[T, 1]`), neg `[T, C]`, cand_ids `[C]`, target_ids `[T]`, weights `[T]` →
  (weighted mean negative log-likelihood of the positive, weighted hit@1).  A candidate equal to the
  row's target is ignored for that row."""
  if not neg.is_cuda:
    return reference(pos, neg, cand_ids, target_ids, weights, temperature)
  return _Fn.apply(pos, neg, cand_ids, target_ids, weights, temperature)
