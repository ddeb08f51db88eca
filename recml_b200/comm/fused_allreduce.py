"""Gradient averaging with the fused NVLink all-reduce (`csrc/cuda/allreduce.cu`).

Gradients are grouped into buckets of ≤64 tensors / `bucket_elems` elements.  Each bucket runs
pack (fp32→bf16 into symmetric memory) → two-shot reduce over peer pointers with the 1/W scale
fused → unpack, on a side stream that starts as soon as the main stream has produced the
gradients, so the exchange overlaps whatever the main stream does next.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch
import torch.distributed as dist

from recml_b200.comm import symm
from recml_b200.ops import _lib

MAXW, MAXT = 8, 64
c_ll, c_vp = ctypes.c_longlong, ctypes.c_void_p


class _Bucket(ctypes.Structure):
  _fields_ = [("grad", c_vp * MAXT), ("numel", c_ll * MAXT), ("offset", c_ll * MAXT),
              ("block_start", c_ll * (MAXT + 1)), ("n", ctypes.c_int)]


class _SeqRef(ctypes.Structure):
  _fields_ = [("ptr", c_vp), ("mul", ctypes.c_ulonglong), ("add", ctypes.c_ulonglong),
              ("literal", ctypes.c_ulonglong)]


class _Comm(ctypes.Structure):
  _fields_ = [("inp", c_vp * MAXW), ("out", c_vp * MAXW), ("flag_a", c_vp * MAXW), ("flag_b", c_vp * MAXW),
              ("my_flag_a", c_vp), ("my_flag_b", c_vp), ("done_counter", c_vp), ("W", ctypes.c_int),
              ("me", ctypes.c_int), ("seq", _SeqRef), ("total", c_ll), ("scale", ctypes.c_float),
              ("status", c_vp), ("mc_in", c_vp), ("mc_out", c_vp)]


class FusedNvlinkReducer:
  def __init__(self, group, device: torch.device, bucket_elems: int = 8 << 20, average: bool = True,
               use_nvls: bool | None = None):
    self.group, self.device = group, device
    # in-switch reduction when asked for (RECML_NVLS=1) and the symmetric buffer has a multicast mapping;
    # NCCL_NVLS_ENABLE=0 turns it off together with NCCL's own NVLS use
    self.use_nvls = symm.nvls_enabled() if use_nvls is None else bool(use_nvls)
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    if self.world > MAXW:
      raise ValueError(f"at most {MAXW} ranks per node")
    self.lib = _lib.cuda()
    sizes = (ctypes.c_int * 2)()
    self.lib.recml_ar_struct_sizes(sizes)
    assert sizes[0] == ctypes.sizeof(_Bucket) and sizes[1] == ctypes.sizeof(_Comm), list(sizes)
    self.bucket_elems = bucket_elems
    self.average = average
    self.cap = 0
    self.buf = None
    self.seq = 0
    self.done = torch.zeros(4, dtype=torch.int32, device=device)
    self.calls = 0                      # host mirror of `calls_dev`
    self.calls_dev = torch.zeros(1, dtype=torch.int64, device=device)
    self.buckets_done = 0               # buckets issued so far (buffer parity)
    self.side = torch.cuda.Stream(device=device)
    self.status = _lib.status_buffer(device)
    self._last_buckets = 0
    self._issued = 0
    self._attached = None
    from recml_b200.utils import graphs
    graphs.register(self)

  def graph_snapshot(self):
    return (self.calls, self.buckets_done)

  def graph_restore(self, snap) -> None:
    self.calls, self.buckets_done = snap

  def graph_advance(self) -> None:
    self.calls += 1
    self.buckets_done += self._last_buckets

  def _ensure(self, elems: int):
    unit = 8 * self.world
    elems = (elems + unit - 1) // unit * unit
    if self.buf is not None and elems <= self.cap:
      return
    cap = torch.tensor([elems], device=self.device, dtype=torch.int64)
    dist.all_reduce(cap, op=dist.ReduceOp.MAX, group=self.group)
    self.cap = int(cap.item())
    cv = symm.Carver()
    self.flag_off = cv.take(2 * MAXW * 8)
    self.in_off = [cv.take(self.cap * 2) for _ in range(2)]
    self.out_off = [cv.take(self.cap * 2) for _ in range(2)]
    self.buf = symm.SymmBuffer(cv.off, self.group, self.device)
    self.seq = 0

  # ---- bucket layout ------------------------------------------------------------------------
  def _layout(self, tensors) -> list[tuple[list, int]]:
    """Greedy buckets of (tensor, element offset) in the given order; offsets are 8-aligned."""
    buckets, cur, n = [], [], 0
    for t in tensors:
      sz = (t.numel() + 7) // 8 * 8
      if cur and (n + sz > self.bucket_elems or len(cur) == MAXT):
        buckets.append((cur, n)); cur, n = [], 0
      cur.append((t, n)); n += sz
    if cur:
      buckets.append((cur, n))
    if len(buckets) > 64:
      raise ValueError("more than 64 gradient buckets; raise bucket_elems")
    return buckets

  def _begin(self, producer: torch.cuda.Stream) -> None:
    """First bucket of a step: fork the side stream off `producer` and advance the call counter."""
    self.side.wait_stream(producer)
    self.calls += 1
    self._issued = 0
    with torch.cuda.stream(self.side):
      _lib.check_rc(self.lib.recml_tick(_lib.ptr(self.calls_dev), ctypes.c_void_p(self.side.cuda_stream)), "tick")

  def _issue(self, items, n: int) -> None:
    """Launches pack + two-shot reduce + unpack of one bucket on the side stream.  `items` is a list
    of (fp32 gradient, element offset); the k-th bucket issued in call c signals c*64 + k, which is
    monotonic because every rank issues its buckets in the same order."""
    k = self._issued
    self._issued += 1
    par = self.buckets_done & 1
    self.buckets_done += 1
    unit = 8 * self.world
    total = (n + unit - 1) // unit * unit
    b = _Bucket()
    blocks = 0
    for i, (g, off) in enumerate(items):
      b.grad[i], b.numel[i], b.offset[i] = g.data_ptr(), g.numel(), off
      b.block_start[i] = blocks
      blocks += (g.numel() + 2047) // 2048
    b.block_start[len(items)] = blocks
    b.n = len(items)
    c = _Comm()
    for r in range(self.world):
      c.inp[r] = self.buf.peer_ptr(r, self.in_off[par])
      c.out[r] = self.buf.peer_ptr(r, self.out_off[par])
      c.flag_a[r] = self.buf.peer_ptr(r, self.flag_off + self.rank * 8)
      c.flag_b[r] = self.buf.peer_ptr(r, self.flag_off + (MAXW + self.rank) * 8)
    c.my_flag_a = self.buf.peer_ptr(self.rank, self.flag_off)
    c.my_flag_b = self.buf.peer_ptr(self.rank, self.flag_off + MAXW * 8)
    c.done_counter = self.done.data_ptr()
    c.W, c.me, c.total = self.world, self.rank, total
    c.seq = _SeqRef(self.calls_dev.data_ptr(), 64, k, 0)
    c.scale = 1.0 / self.world if self.average else 1.0
    c.status = self.status.data_ptr()
    if self.use_nvls and self.buf.multicast_ptr:
      c.mc_in = self.buf.multicast_ptr + self.in_off[par]
      c.mc_out = self.buf.multicast_ptr + self.out_off[par]
    with torch.cuda.stream(self.side):
      _lib.check_rc(self.lib.recml_allreduce_bucket(ctypes.byref(b), ctypes.byref(c),
                                                    ctypes.c_void_p(self.side.cuda_stream)), "allreduce_bucket")

  @staticmethod
  def _fp32_grad(p: torch.Tensor) -> torch.Tensor:
    g = p.grad
    if g.dtype != torch.float32 or not g.is_contiguous():
      g = g.to(torch.float32).contiguous()
      p.grad = g
    return g

  # ---- overlapped mode: reduce a bucket as soon as backward has produced it ------------------
  def attach(self, params: Sequence[torch.Tensor]) -> None:
    """Fixes the bucket layout over `params` (filled in reverse order, the order in which backward
    produces gradients) and hooks every parameter so that a bucket is reduced on the side stream
    the moment its last gradient has been accumulated; `average_grads` then only launches what is
    left and joins the side stream.  Collective: every rank attaches the same parameters.  One
    backward pass per `average_grads` call (no gradient accumulation across backward passes)."""
    if self._attached is not None:
      if [id(p) for p in self._attached] == [id(p) for p in reversed(list(params))]:
        return
      for h in self._hooks:       # a new state replaces the old one
        h.remove()
    order = [p for p in reversed(list(params))]
    self._attached = order
    self._abuckets = self._layout(order)
    self._bucket_of = {}
    for bi, (items, _) in enumerate(self._abuckets):
      for p, _off in items:
        self._bucket_of[id(p)] = bi
    self._ensure(max(n for _, n in self._abuckets))
    self._reset_step()
    self._hooks = [p.register_post_accumulate_grad_hook(self._on_grad) for p in order]

  def _reset_step(self) -> None:
    self._ready = [0] * len(self._abuckets)
    self._launched = [False] * len(self._abuckets)
    self._began = False

  def _launch_attached(self, bi: int) -> None:
    cur = torch.cuda.current_stream(self.device)
    if not self._began:
      self._began = True
      self._begin(cur)
    else:
      self.side.wait_stream(cur)
    items, n = self._abuckets[bi]
    live = [(self._fp32_grad(p), off) for p, off in items if p.grad is not None]
    self._launched[bi] = True
    if live:
      self._issue(live, n)

  def _on_grad(self, p: torch.Tensor) -> None:
    bi = self._bucket_of[id(p)]
    if self._launched[bi]:
      raise RuntimeError("a gradient arrived for a bucket that was already reduced: overlapped gradient "
                         "reduction supports one backward pass per optimizer step")
    self._ready[bi] += 1
    if self._ready[bi] == len(self._abuckets[bi][0]):
      self._launch_attached(bi)

  def _finish_attached(self, params: Sequence[torch.Tensor]) -> None:
    known = self._bucket_of
    extra = [p for p in params if id(p) not in known]
    if extra:
      raise ValueError(f"{len(extra)} parameters were not attached to the overlapped reducer")
    for bi in range(len(self._abuckets)):
      if not self._launched[bi] and any(p.grad is not None for p, _ in self._abuckets[bi][0]):
        self._launch_attached(bi)
    if self._began:
      torch.cuda.current_stream(self.device).wait_stream(self.side)
    self._last_buckets = self._issued if self._began else 0
    self._reset_step()

  def average_grads(self, params: Sequence[torch.Tensor]) -> None:
    if self._attached is not None:
      self._finish_attached(params)
      return
    grads = [self._fp32_grad(p) for p in params]
    buckets = self._layout(grads)
    self._ensure(max(n for _, n in buckets))
    main = torch.cuda.current_stream(self.device)
    self._begin(main)
    self._last_buckets = len(buckets)
    for items, n in buckets:
      self._issue(items, n)
    main.wait_stream(self.side)
