"""Rank of the target item among the whole (row-sharded) vocabulary without materialising logits.

Every rank scores the query states of ALL ranks against its own item shard (the fused
all-gather → tcgen05 GEMM → count kernel, `csrc/cuda/vocab_rank.cu`) and the per-row counts of
better-scoring items are summed across ranks: rank = 1 + Σ counts.  Recall@K / NDCG@K / MRR follow from
the rank (`recml_b200.metrics.ranking`).  Replaces the `[B, L, V]` reverse-embedding matmul + top-k of the
reference's evaluation (`recml/layers/keras/sasrec.py:163`, `recml/core/metrics/mean_metrics.py:43-65`).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from recml_b200.comm import symm
from recml_b200.ops import _lib

MAXW = 8
c_int, c_vp, c_ll = ctypes.c_int, ctypes.c_void_p, ctypes.c_longlong


class _SeqRef(ctypes.Structure):
  _fields_ = [("ptr", c_vp), ("mul", ctypes.c_ulonglong), ("add", ctypes.c_ulonglong), ("literal", ctypes.c_ulonglong)]


class _Params(ctypes.Structure):
  _fields_ = [("M", c_int), ("D", c_int), ("V_local", c_int), ("W", c_int), ("me", c_int), ("rows_per_rank", c_int),
              ("id_mul", c_int), ("id_add", c_int), ("peer_x", c_vp * MAXW), ("stage", c_vp), ("ready_flags", c_vp),
              ("seq", _SeqRef), ("src_done", c_vp), ("pos_score", c_vp), ("target", c_vp), ("count", c_vp),
              ("status", c_vp)]


class _PublishArgs(ctypes.Structure):
  _fields_ = [("flags", c_vp * MAXW)]


def counts_reference(x_all: torch.Tensor, shard: torch.Tensor, pos: torch.Tensor, target: torch.Tensor, id_mul: int,
                     id_add: int) -> torch.Tensor:
  """fp32 oracle: x_all `[M, D]`, shard `[V_l, D]`."""
  s = x_all.float() @ shard.float().t()
  ids = torch.arange(shard.shape[0], device=s.device) * id_mul + id_add
  better = (s > pos[:, None]) & (ids[None, :] != target[:, None])
  return better.sum(dim=1).to(torch.int32)


class VocabRanker:
  """Workspace + driver.  `rows` = query rows per rank per call (fixed), `dim` = embedding dim."""

  def __init__(self, rows: int, dim: int, group=None, device: torch.device | None = None):
    self.group = group
    self.world = symm.world_of(group)
    self.rank = dist.get_rank(group) if self.world > 1 else 0
    self.device = device or torch.device("cuda", torch.cuda.current_device())
    self.rows, self.dim = rows, dim
    self.cuda = self.device.type == "cuda"
    self.calls = 0
    if not self.cuda:
      return
    if rows * self.world > 4096:
      raise ValueError("at most 4096 query rows per call across all ranks")
    self.lib = _lib.cuda()
    assert int(self.lib.recml_vocab_rank_struct_size()) == ctypes.sizeof(_Params)
    cv = symm.Carver()
    self.flag_off = cv.take(MAXW * 8)
    self.x_off = [cv.take(rows * dim * 2) for _ in range(2)]
    self.buf = symm.SymmBuffer(cv.off, group, self.device)
    self.stage = torch.empty(rows * self.world, dim, dtype=torch.bfloat16, device=self.device)
    self.src_done = torch.zeros(MAXW, dtype=torch.int32, device=self.device)
    self.calls_dev = torch.zeros(1, dtype=torch.int64, device=self.device)

  def counts(self, x: torch.Tensor, pos_all: torch.Tensor, target_all: torch.Tensor, shard_bf16: torch.Tensor,
             id_mul: int, id_add: int) -> torch.Tensor:
    """x `[rows, D]` this rank's query states; pos_all / target_all `[rows·W]` for all ranks (rank-major);
    returns this rank's `[rows·W]` int32 counts over ITS shard."""
    W, M = self.world, self.rows * self.world
    if not self.cuda:
      xs = [torch.empty_like(x) for _ in range(W)]
      if W > 1:
        dist.all_gather(xs, x.contiguous(), group=self.group)
      else:
        xs = [x]
      return counts_reference(torch.cat(xs), shard_bf16, pos_all, target_all, id_mul, id_add)
    self.calls += 1
    par = self.calls & 1
    st = _lib.stream()
    _lib.check_rc(self.lib.recml_tick(_lib.ptr(self.calls_dev), st), "tick")
    seq = _SeqRef(self.calls_dev.data_ptr(), 1, 0, 0)
    xbuf = self.buf.view(self.x_off[par], (self.rows, self.dim), torch.bfloat16)
    xbuf.copy_(x.to(torch.bfloat16))
    if W > 1:
      pa = _PublishArgs()
      for r in range(W):
        pa.flags[r] = self.buf.peer_ptr(r, self.flag_off + self.rank * 8)
      _lib.check_rc(self.lib.recml_publish_flags(ctypes.byref(pa), c_int(W), ctypes.byref(seq), st), "publish")
    count = torch.zeros(M, dtype=torch.int32, device=self.device)
    self.src_done.zero_()
    p = _Params()
    p.M, p.D, p.V_local, p.W, p.me, p.rows_per_rank = M, self.dim, shard_bf16.shape[0], W, self.rank, self.rows
    p.id_mul, p.id_add = id_mul, id_add
    for r in range(W):
      p.peer_x[r] = self.buf.peer_ptr(r, self.x_off[par])
    p.stage = self.stage.data_ptr()
    p.ready_flags = self.buf.peer_ptr(self.rank, self.flag_off) if W > 1 else None
    p.seq = seq
    p.src_done, p.pos_score = self.src_done.data_ptr(), pos_all.float().contiguous().data_ptr()
    tgt = target_all.to(torch.int64).contiguous()
    pos = pos_all.float().contiguous()
    p.pos_score, p.target, p.count = pos.data_ptr(), tgt.data_ptr(), count.data_ptr()
    p.status = _lib.status_buffer(self.device).data_ptr()
    assert shard_bf16.dtype == torch.bfloat16 and shard_bf16.is_contiguous()
    _lib.check_rc(self.lib.recml_vocab_rank(_lib.ptr(shard_bf16), ctypes.byref(p), st), "vocab_rank")
    return count

  def ranks(self, x: torch.Tensor, pos: torch.Tensor, target: torch.Tensor, shard_bf16: torch.Tensor, id_mul: int,
            id_add: int) -> torch.Tensor:
    """1-based rank of each local row's target over the whole vocabulary."""
    W = self.world
    if W > 1:
      pos_all = torch.empty(self.rows * W, dtype=torch.float32, device=x.device)
      tgt_all = torch.empty(self.rows * W, dtype=torch.int64, device=x.device)
      dist.all_gather_into_tensor(pos_all, pos.float().contiguous(), group=self.group)
      dist.all_gather_into_tensor(tgt_all, target.to(torch.int64).contiguous(), group=self.group)
    else:
      pos_all, tgt_all = pos.float(), target.to(torch.int64)
    cnt = self.counts(x, pos_all, tgt_all, shard_bf16, id_mul, id_add)
    if W > 1:
      dist.all_reduce(cnt, group=self.group)
    return 1 + cnt[self.rank * self.rows:(self.rank + 1) * self.rows].to(torch.int64)
