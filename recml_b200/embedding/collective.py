"""Sharded-embedding backend built from torch ops and `torch.distributed` collectives.

Used (a) on CPU with gloo for multi-process tests, (b) as the oracle for the fused
kernels and (c) on GPU with NCCL as the "library path" stand-in baseline.  It follows
the same three exchanges as the fused backend: ids are all-gathered, every owner pools
what it owns for ALL samples of the job, partial results travel back with an all-to-all
and are summed at the destination; backward all-gathers the activation gradients and
each owner aggregates per unique row and applies the row optimizer.
"""
from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from recml_b200.embedding import jagged as jagged_lib
from recml_b200.embedding import row_optim
from recml_b200.embedding.planner import Placement


def feature_layout(module) -> tuple[list[tuple[str, int, int, int]], int]:
  """[(feature, col offset, width, seq len or 0)] for sharded features, total width."""
  cols, off = [], 0
  for f in module.feature_names:
    spec = module.config.specs[f]
    if module.plan.tables[module.feature_to_table[f]].placement is Placement.REPLICATED:
      continue
    L = spec.max_sequence_length or 0
    width = spec.embedding_dim * max(L, 1)
    cols.append((f, off, width, L))
    off += width
  return cols, off


def bag_gains(spec, lens: torch.Tensor, bag: torch.Tensor, w: torch.Tensor | None) -> torch.Tensor:
  """Per-id multiplier implementing the combiner (sum / mean / sqrtn), weighted or not."""
  n = bag.numel()
  w = torch.ones(n, device=bag.device) if w is None else w.to(torch.float32)
  if spec.max_sequence_length is not None or spec.combiner == "sum":
    return w
  B = lens.numel()
  if spec.combiner == "mean":
    den = torch.zeros(B, device=bag.device).index_add_(0, bag, w)
  else:
    den = torch.sqrt(torch.zeros(B, device=bag.device).index_add_(0, bag, w * w))
  den = torch.where(den == 0, torch.ones_like(den), den)
  return w / den[bag]


class CollectiveBackend:
  def __init__(self, module):
    self.m = module
    self.layout, self.width = feature_layout(module)

  # -- helpers ----------------------------------------------------------------------------
  def _gather_kjt(self, kjt: jagged_lib.KeyedJagged):
    """All ranks' (values, offsets, weights) lists, rank-major."""
    m = self.m
    if m.world == 1:
      return [(kjt.values, kjt.offsets, kjt.weights)]
    dev = kjt.values.device
    n = torch.tensor([kjt.values.numel()], device=dev, dtype=torch.int64)
    ns = [torch.zeros_like(n) for _ in range(m.world)]
    dist.all_gather(ns, n, group=m.group)
    nmax = int(max(int(x) for x in ns))
    pad = torch.zeros(max(nmax, 1), dtype=kjt.values.dtype, device=dev)
    pad[:kjt.values.numel()] = kjt.values
    vals = [torch.empty_like(pad) for _ in range(m.world)]
    dist.all_gather(vals, pad, group=m.group)
    offs = [torch.empty_like(kjt.offsets) for _ in range(m.world)]
    dist.all_gather(offs, kjt.offsets.contiguous(), group=m.group)
    ws = [None] * m.world
    if kjt.weights is not None:
      padw = torch.zeros(max(nmax, 1), dtype=torch.float32, device=dev)
      padw[:kjt.weights.numel()] = kjt.weights
      ws = [torch.empty_like(padw) for _ in range(m.world)]
      dist.all_gather(ws, padw, group=m.group)
    return [(vals[r][:int(ns[r])], offs[r], None if ws[r] is None else ws[r][:int(ns[r])])
            for r in range(m.world)]

  def _local_rows(self, tp, ids: torch.Tensor):
    """(owned mask, row index inside the stack) for global ids of one table."""
    m = self.m
    if tp.placement is Placement.ROW_WISE:
      owned = (ids % m.world + tp.rotation) % m.world == m.rank
      return owned, tp.row_base + ids // m.world
    if tp.placement is Placement.TABLE_WISE:
      owned = torch.full_like(ids, tp.owner == m.rank, dtype=torch.bool)
      return owned, tp.row_base + ids
    return torch.ones_like(ids, dtype=torch.bool), tp.row_base + ids  # COLUMN_WISE

  # -- forward -------------------------------------------------------------------------------
  def forward(self, kjt: jagged_lib.KeyedJagged, training: bool, out=None, out_col: int = 0):
    m = self.m
    B, W, F = kjt.batch_size(), m.world, len(m.feature_names)
    dev = m.device
    parts = self._gather_kjt(kjt)
    send = torch.zeros(W * B, self.width, dtype=torch.float32, device=dev)
    saved = []
    for fname, col, width, L in self.layout:
      spec = m.config.specs[fname]
      tp = m.plan.tables[m.feature_to_table[fname]]
      fi = m.feature_names.index(fname)
      ids_l, bag_l, gain_l = [], [], []
      for s, (vals, offs, w) in enumerate(parts):
        o = offs[fi * B:(fi + 1) * B + 1].to(torch.int64)
        a, b = int(o[0]), int(o[-1])
        lens = o[1:] - o[:-1]
        bag = torch.repeat_interleave(torch.arange(B, device=dev), lens)
        ids = vals[a:b].to(torch.int64)
        gains = bag_gains(spec, lens, bag, None if w is None else w[a:b])
        if L:
          pos = torch.arange(b - a, device=dev) - (o[:-1] - a)[bag]
          keep = pos < L
          ids, gains = ids[keep], gains[keep]
          bag = (s * B + bag[keep]) * L + pos[keep]
        else:
          bag = s * B + bag
        ids_l.append(ids); bag_l.append(bag); gain_l.append(gains)
      ids, bag, gains = torch.cat(ids_l), torch.cat(bag_l), torch.cat(gain_l)
      owned, rows = self._local_rows(tp, ids)
      rows, bag_o, gains_o = rows[owned], bag[owned], gains[owned]
      D = tp.local_dim
      vec = m.stack_weights[tp.stack][rows] * gains_o[:, None]
      nb = W * B * max(L, 1)
      pooled = torch.zeros(nb, D, device=dev).index_add_(0, bag_o, vec)
      if tp.placement is Placement.COLUMN_WISE:
        full = torch.zeros(nb, tp.dim, device=dev)
        full[:, tp.col_lo:tp.col_lo + D] = pooled
        pooled = full
      send[:, col:col + width] = pooled.reshape(W * B, width)
      if training:
        saved.append((tp, col, width, L, rows, bag_o, gains_o))
    if W > 1:
      recv = torch.empty_like(send)
      dist.all_to_all_single(recv, send, group=m.group)
      out_sum = recv.view(W, B, self.width).sum(dim=0)
    res = send if W == 1 else out_sum
    if out is not None:
      out[:, out_col:out_col + self.width] = res.to(out.dtype)
      res = out[:, out_col:out_col + self.width]
    elif m.config.output_dtype is not None:
      res = res.to(m.config.output_dtype)
    return res, (saved if training else None)

  # -- backward: aggregate per unique row inside each stack, then update ---------------------------
  @torch.no_grad()
  def backward(self, saved: Any, grad_out: torch.Tensor) -> None:
    m = self.m
    W = m.world
    g = grad_out.to(torch.float32).contiguous()
    if W > 1:
      parts = [torch.empty_like(g) for _ in range(W)]
      dist.all_gather(parts, g, group=m.group)
      g = torch.cat(parts, dim=0)
    per_stack: dict[int, list[tuple[torch.Tensor, torch.Tensor]]] = {}
    for tp, col, width, L, rows, bag, gains in saved:
      D = tp.dim
      gf = g[:, col:col + width].reshape(-1, D)[bag]
      if tp.placement is Placement.COLUMN_WISE:
        gf = gf[:, tp.col_lo:tp.col_lo + tp.local_dim]
      per_stack.setdefault(tp.stack, []).append((rows, gf * gains[:, None]))
    for si, items in per_stack.items():
      rows = torch.cat([r for r, _ in items])
      if rows.numel() == 0:
        continue
      grads = torch.cat([x for _, x in items])
      uniq, inv = torch.unique(rows, return_inverse=True)
      agg = torch.zeros(uniq.numel(), grads.shape[1], device=grads.device).index_add_(0, inv, grads)
      agg *= m.grad_scale
      opt = m.plan.stacks[si].optimizer
      slots = {k: v[uniq] for k, v in m.stack_slots[si].items()}
      new_w, new_slots = row_optim.apply(opt, m.step_count, m.stack_weights[si][uniq], agg, slots)
      m.stack_weights[si][uniq] = new_w
      for k, v in new_slots.items():
        m.stack_slots[si][k][uniq] = v
