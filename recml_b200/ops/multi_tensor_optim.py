"""Fused dense optimizer step (`csrc/cuda/optim.cu`): one launch per ≤64 tensors performs
global-norm clipping, Adam / RSS / SGD scaling, masked weight decay, the learning-rate step and
refreshes the bf16 compute copy attached to a parameter (`param._recml_bf16`)."""
from __future__ import annotations

import ctypes

import torch

from recml_b200.ops import _lib

MAX_T = 64


class _TensorList(ctypes.Structure):
  _fields_ = [("param", ctypes.c_void_p * MAX_T), ("grad", ctypes.c_void_p * MAX_T),
              ("s0", ctypes.c_void_p * MAX_T), ("s1", ctypes.c_void_p * MAX_T),
              ("copy", ctypes.c_void_p * MAX_T), ("numel", ctypes.c_longlong * MAX_T),
              ("block_start", ctypes.c_longlong * (MAX_T + 1)), ("decay", ctypes.c_int * MAX_T),
              ("n", ctypes.c_int)]


class _Hyper(ctypes.Structure):
  _fields_ = [("kind", ctypes.c_int), ("lr", ctypes.c_float), ("b1", ctypes.c_float), ("b2", ctypes.c_float),
              ("eps", ctypes.c_float), ("bc1", ctypes.c_float), ("bc2", ctypes.c_float),
              ("weight_decay", ctypes.c_float), ("clip_norm", ctypes.c_float), ("sqnorm", ctypes.c_void_p)]


_checked = False


def _check_layout(lib):
  global _checked
  if not _checked:
    sizes = (ctypes.c_int * 2)()
    lib.recml_optim_struct_sizes(sizes)
    assert sizes[0] == ctypes.sizeof(_TensorList) and sizes[1] == ctypes.sizeof(_Hyper), \
        (list(sizes), ctypes.sizeof(_TensorList), ctypes.sizeof(_Hyper))
    _checked = True


RING = 512


def _hyper_for(opt, lr: float, t: int, sq_ptr) -> _Hyper:
  kind = {"identity": 0, "adam": 1, "rss": 2}[opt.scaling.kind]
  return _Hyper(kind, lr, opt.scaling.b1, opt.scaling.b2, opt.scaling.eps, 1.0 - opt.scaling.b1 ** t,
                1.0 - opt.scaling.b2 ** t, opt.weight_decay or 0.0, opt.grad_clip_norm or 0.0, sq_ptr)


def push_hyper(opt, lr: float, t: int) -> None:
  """Writes the step's hyper-parameters into the optimizer's device struct (stream-ordered copy
  from a ring of pinned slots, so the host may run ahead of the GPU)."""
  if not hasattr(opt, "_hyper_dev"):
    dev = opt.params[0].device
    opt._hyper_dev = torch.zeros(ctypes.sizeof(_Hyper), dtype=torch.uint8, device=dev)
    opt._hyper_ring = torch.zeros(RING, ctypes.sizeof(_Hyper), dtype=torch.uint8).pin_memory()
    opt._hyper_slot = 0
    opt._sq = torch.zeros(1, dtype=torch.float32, device=dev)
  h = _hyper_for(opt, lr, t, opt._sq.data_ptr() if opt.grad_clip_norm is not None else None)
  slot = opt._hyper_ring[opt._hyper_slot % RING]
  opt._hyper_slot += 1
  ctypes.memmove(slot.data_ptr(), ctypes.addressof(h), ctypes.sizeof(_Hyper))
  opt._hyper_dev.copy_(slot, non_blocking=True)


def fused_step(opt, live: list[int], grads: list[torch.Tensor], lr: float):
  """Runs the update for `opt` (an `optim_factory.Optimizer`) on CUDA; returns the grad norm
  tensor when clipping is on.  Hyper-parameters are read by the kernel from device memory, so the
  same launch sequence is valid inside a captured CUDA graph."""
  from recml_b200.utils import graphs
  lib = _lib.cuda()
  _check_layout(lib)
  kind = {"identity": 0, "adam": 1, "rss": 2}[opt.scaling.kind]
  t = opt.count + 1
  if not graphs.capturing():
    push_hyper(opt, lr, t)       # during capture the copy is issued by graph_pre_replay instead
  grads = [g if (g.dtype == torch.float32 and g.is_contiguous()) else g.to(torch.float32).contiguous()
           for g in grads]
  lists = []
  for a in range(0, len(live), MAX_T):
    tl = _TensorList()
    blocks = 0
    idx = live[a:a + MAX_T]
    for j, i in enumerate(idx):
      p = opt.params[i]
      assert p.dtype == torch.float32 and p.is_contiguous(), "fused optimizer needs fp32 contiguous params"
      tl.param[j] = p.data_ptr()
      tl.grad[j] = grads[a + j].data_ptr()
      if kind == 1:
        tl.s0[j], tl.s1[j] = opt.slots["mu"][i].data_ptr(), opt.slots["nu"][i].data_ptr()
      elif kind == 2:
        tl.s0[j] = opt.slots["sum_of_squares"][i].data_ptr()
      cp = getattr(p, "_recml_bf16", None)
      tl.copy[j] = cp.data_ptr() if cp is not None else None
      tl.numel[j] = p.numel()
      tl.block_start[j] = blocks
      blocks += (p.numel() + 1023) // 1024
      tl.decay[j] = int(opt.decay_flags[i])
    tl.block_start[len(idx)] = blocks
    tl.n = len(idx)
    lists.append(tl)
  sq = None
  if opt.grad_clip_norm is not None:
    sq = opt._sq
    sq.zero_()
    for tl in lists:
      _lib.check_rc(lib.recml_optim_sqnorm(ctypes.byref(tl), _lib.ptr(sq), _lib.stream()), "optim_sqnorm")
  h = _hyper_for(opt, lr, t, None)
  for tl in lists:
    _lib.check_rc(lib.recml_optim_step(ctypes.byref(tl), ctypes.byref(h), _lib.ptr(opt._hyper_dev),
                                       _lib.stream()), "optim_step")
  for i in live:
    p = opt.params[i]
    if getattr(p, "_recml_bf16", None) is not None:
      p._recml_bf16_version = p._version
  return None if sq is None else sq.sqrt()
