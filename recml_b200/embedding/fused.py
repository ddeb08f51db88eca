"""Fused sharded-embedding backend: sm_100a kernels over NVLink peer memory
(`csrc/cuda/embedding.cu`, `csrc/cuda/radix_sort.cu`).

Per step:  ids are pushed to every peer (one kernel, peer stores + flag) → one forward kernel per
table stack gathers / pools the rows this rank owns for EVERY rank's samples and stores each
pooled bf16 vector straight into the requesting rank's buffer (the all-to-all is the store) →
the combine kernel waits for all sources' flags, sums the per-source slots of row-sharded
features and writes the concatenated dense input.  The (row, gradient index) occurrences recorded
by the forward are radix-sorted by row on a side stream while the dense forward runs.  Backward
(on its own side stream, beside the dense weight-gradient GEMMs): one kernel pushes each feature's
activation gradient into its owner's buffer, the owner reduces runs of equal rows of the sorted
occurrences and applies the row optimizer inside the same kernel.  All buffers that peers write
are double-buffered by step parity; flags are monotonically increasing step sequence numbers, and
every wait is bounded.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

import torch

from recml_b200.comm import symm
from recml_b200.embedding import collective
from recml_b200.embedding import jagged as jagged_lib
from recml_b200.embedding.planner import Placement
from recml_b200.ops import _lib
from recml_b200.utils import streams

MAXW = 8
c_ll, c_int, c_uint, c_float, c_vp = (ctypes.c_longlong, ctypes.c_int, ctypes.c_uint, ctypes.c_float,
                                      ctypes.c_void_p)
KIND = {Placement.TABLE_WISE: 0, Placement.ROW_WISE: 1, Placement.COLUMN_WISE: 2}
COMBINER = {"sum": 0, "mean": 1, "sqrtn": 2}
OPT = {"sgd": 0, "adagrad": 1, "rowwise_adagrad": 2, "adam": 3, "rowwise_adam": 4,
       "adagrad_momentum": 5, "ftrl": 6, "laprop": 7}


class SeqRef(ctypes.Structure):
  """Sequence number of a flag exchange: `*ptr * mul + add` when ptr is set, else `literal`."""
  _fields_ = [("ptr", c_vp), ("mul", ctypes.c_ulonglong), ("add", ctypes.c_ulonglong),
              ("literal", ctypes.c_ulonglong)]


class FeatDesc(ctypes.Structure):
  _fields_ = [("feat_index", c_int), ("kind", c_int), ("owner", c_int), ("rot", c_int), ("row_base", c_int),
              ("combiner", c_int), ("dim", c_int), ("col_lo", c_int), ("slot_off", c_ll), ("grad_off", c_ll),
              ("seq_len", c_int), ("dst_stride", c_int), ("vocab", c_int), ("tile_shift", c_int),
              ("tile_start", c_ll)]


class IdPtrs(ctypes.Structure):
  _fields_ = [("values", c_vp * MAXW), ("offsets", c_vp * MAXW), ("weights", c_vp * MAXW)]


class FwdParams(ctypes.Structure):
  _fields_ = [("ids", IdPtrs), ("feats", c_vp), ("n_feats", c_int), ("W", c_int), ("me", c_int), ("B", c_int),
              ("dloc", c_int), ("table", c_vp), ("pooled", c_vp * MAXW), ("occ_key", c_vp), ("occ_val", c_vp),
              ("occ_gain", c_vp), ("occ_count", c_vp), ("occ_cap", c_uint), ("grad_ld", c_ll), ("wait_flags", c_vp),
              ("done_counter", c_vp), ("flags", c_vp * MAXW), ("seq", SeqRef), ("status", c_vp), ("dropped", c_vp),
              ("prefetch", c_int), ("tiled", c_int), ("total_tiles", c_ll), ("prefiltered", c_int)]


class CombineDesc(ctypes.Structure):
  _fields_ = [("slot_off", c_ll), ("nslots", c_int), ("dim", c_int), ("out_col", c_int), ("seq_len", c_int),
              ("rw_index", c_int), ("pad", c_int)]


class CombineParams(ctypes.Structure):
  _fields_ = [("pooled", c_vp), ("feats", c_vp), ("n_feats", c_int), ("B", c_int), ("out", c_vp), ("ld_out", c_ll),
              ("wait_flags", c_vp), ("W", c_int), ("n_chan", c_int), ("seq", SeqRef), ("status", c_vp),
              ("cnt_raw", c_vp)]


class PushGradDesc(ctypes.Structure):
  _fields_ = [("kind", c_int), ("owner", c_int), ("dim", c_int), ("in_col", c_int), ("seq_len", c_int),
              ("rw_index", c_int), ("grad_off", c_ll * MAXW)]


class PushGradParams(ctypes.Structure):
  _fields_ = [("grad", c_vp), ("ld", c_ll), ("feats", c_vp), ("n_feats", c_int), ("B", c_int), ("W", c_int),
              ("me", c_int), ("dst", c_vp * MAXW), ("done_counter", c_vp), ("flags", c_vp * MAXW),
              ("seq", SeqRef), ("cnt_raw", c_vp)]


class BwdParams(ctypes.Structure):
  _fields_ = [("keys", c_vp), ("vals", c_vp), ("occ_gain", c_vp), ("n_occ", c_vp), ("grads", c_vp), ("val_scale", c_ll),
              ("table", c_vp), ("slot0", c_vp), ("slot1", c_vp), ("dloc", c_int), ("opt", c_int),
              ("hp", c_float * 6), ("grad_scale", c_float), ("slot1_rowwise", c_int), ("scratch", c_vp),
              ("wait_flags", c_vp), ("W", c_int), ("seq", SeqRef), ("status", c_vp), ("hp_dev", c_vp),
              ("n_cap", c_uint), ("reserved", c_int)]


class PushIdsParams(ctypes.Structure):
  _fields_ = [("values", c_vp), ("offsets", c_vp), ("weights", c_vp), ("nnz", c_ll), ("n_offsets", c_int),
              ("W", c_int), ("me", c_int), ("dst_values", c_vp * MAXW), ("dst_offsets", c_vp * MAXW),
              ("dst_weights", c_vp * MAXW), ("done_counter", c_vp), ("flags", c_vp * MAXW),
              ("seq", SeqRef), ("need", c_vp), ("n_feats", c_int), ("B", c_int)]


class BucketFeat(ctypes.Structure):
  _fields_ = [("kind", c_int), ("owner", c_int), ("rot", c_int), ("rw_index", c_int)]


class BucketizeParams(ctypes.Structure):
  _fields_ = [("values", c_vp), ("offsets", c_vp), ("weights", c_vp), ("n_feats", c_int), ("B", c_int), ("W", c_int),
              ("me", c_int), ("n_rw", c_int), ("feats", c_vp), ("cnt", c_vp), ("tot", c_vp), ("cnt_raw", c_vp),
              ("dst_values", c_vp * MAXW), ("dst_offsets", c_vp * MAXW), ("dst_weights", c_vp * MAXW),
              ("done_counter", c_vp), ("flags", c_vp * MAXW), ("seq", SeqRef)]


_layout_checked = False


def _check_layout(lib):
  global _layout_checked
  if _layout_checked:
    return
  sizes = (c_int * 8)()
  lib.recml_emb_struct_sizes(sizes)
  mine = [ctypes.sizeof(t) for t in (FeatDesc, FwdParams, CombineDesc, CombineParams, PushGradDesc,
                                     PushGradParams, BwdParams, PushIdsParams)]
  assert list(sizes) == mine, f"struct layout mismatch: C {list(sizes)} vs ctypes {mine}"
  assert int(lib.recml_emb_bucketize_struct_size()) == ctypes.sizeof(BucketizeParams)
  _layout_checked = True


def _device_struct_array(items, device) -> torch.Tensor:
  if not items:
    return torch.zeros(8, dtype=torch.uint8, device=device)
  raw = b"".join(bytes(x) for x in items)
  return torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)


class FusedBackend:
  """See the module docstring.  Buffers are sized lazily from the first batch
  (`capacity_factor` × its id count) and grown when a later batch needs more."""

  def __init__(self, module, capacity_factor: float = 1.25):
    self.m = module
    self.lib = _lib.cuda()
    _check_layout(self.lib)
    m = module
    if m.world > MAXW:
      raise ValueError(f"fused backend supports up to {MAXW} ranks per node, got {m.world}")
    self.layout, self.width = collective.feature_layout(m)
    self.capacity_factor = capacity_factor
    self.seq = 0
    self._need = None
    self.seq_dev = torch.zeros(1, dtype=torch.int64, device=module.device)
    self.B = None
    self.status = _lib.status_buffer(m.device)
    # resident 128-thread blocks per SM of the backward update kernel: 0 = fill the GPU; a model that runs
    # weight-gradient GEMMs beside the embedding backward sets -1 so that a GEMM CTA fits on every SM
    self.bwd_blocks_per_sm = int(os.environ.get("RECML_EMB_BWD_BLOCKS", "0"))
    self.side_streams = os.environ.get("RECML_EMB_STREAMS", "1") != "0"
    self.fwd_prefetch = int(os.environ.get("RECML_EMB_FWD_PREFETCH", "3"))    # bit 0: L2 prefetch, bit 1: id queue
    self.fwd_tiled = os.environ.get("RECML_EMB_FWD_TILED", "1") != "0"
    # Senders sort the ids of row-sharded pooled features by owning rank, so that a rank receives (and scans)
    # only its own; needs whole-bag combiner denominators to be unnecessary, i.e. sum combiners on those features.
    self.bucketize = os.environ.get("RECML_EMB_BUCKETIZE", "1") != "0"
    self._bucket = None
    self.dropped = torch.zeros(1, dtype=torch.int32, device=module.device) if module.config.allow_id_dropping else None
    # lookups that may be in flight before their update runs: 1 for the ordinary step; 2 under software
    # pipelining (`training/pipeline.py`), where lookup(i + 1) precedes update(i).  Each in-flight lookup has
    # its own occurrence list, and sequence numbers are launch-time literals (the device-side counter, which
    # exists for CUDA-graph replay, would have moved on by the time a delayed backward reads it).
    self.pipeline_depth = 1
    self._train_calls = 0
    self._hp_slot = 0
    from recml_b200.utils import graphs
    graphs.register(self)
    self.has_gains = any(s.combiner != "sum" or s.weight_name is not None
                         for s in m.config.specs.values())

  # -- CUDA-graph protocol: host mirrors of device-side counters ----------------------------------------
  def graph_snapshot(self):
    return (self.seq, self.m.step_count)

  def graph_restore(self, snap) -> None:
    self.seq, self.m.step_count = snap

  def graph_advance(self) -> None:
    self.seq += 1
    self.m.step_count += 1

  def graph_pre_replay(self) -> None:
    self._push_hyper()

  def set_pipeline_depth(self, depth: int) -> None:
    if self._occ_ready_flag():
      raise RuntimeError("set the pipeline depth before the first training lookup")
    self.pipeline_depth = int(depth)

  def _occ_ready_flag(self) -> bool:
    return bool(getattr(self, "_occ_ready", False))

  # -- row-optimizer hyper-parameters live on the device (a replayed graph follows a schedule) -----------
  HP_RING = 256

  def _push_hyper(self) -> None:
    """Copies this step's hyper-parameters of every stack into device memory through a ring of pinned
    slots (stream-ordered, so the host may run ahead of the device)."""
    m = self.m
    if not getattr(self, "_occ_ready", False):
      return
    n = len(self.stacks)
    if not hasattr(self, "_hp_ring"):
      self._hp_ring = torch.zeros(self.HP_RING, n, 8, dtype=torch.float32).pin_memory()
      self._hp_dev = torch.zeros(n, 8, dtype=torch.float32, device=m.device)
    slot = self._hp_ring[self._hp_slot % self.HP_RING]
    self._hp_slot += 1
    for si in range(n):
      hp = m.plan.stacks[si].optimizer.hyperparams(m.step_count)
      for i in range(6):
        slot[si, i] = float(hp[i]) if i < len(hp) else 0.0
    self._hp_dev.copy_(slot, non_blocking=True)

  def dropped_ids(self) -> int:
    """Ids dropped so far because an occurrence list was full (`allow_id_dropping`); synchronises."""
    return 0 if self.dropped is None else int(self.dropped.item())

  # -- one-time set-up for a batch geometry --------------------------------------------------------------
  def _setup(self, kjt: jagged_lib.KeyedJagged):
    m = self.m
    W, B, dev = m.world, kjt.batch_size(), m.device
    self.B = B
    F = len(m.feature_names)
    self.n_offsets = F * B + 1
    # ids per bag of every feature in this first batch (one small read-back at set-up): sizes the forward's tiles
    bounds = kjt.offsets[::B].to(torch.int64).cpu().tolist() if kjt.offsets.numel() == F * B + 1 else None
    self._avg_bag = ({f: (bounds[i + 1] - bounds[i]) / max(B, 1) for i, f in enumerate(m.feature_names)}
                     if bounds is not None and len(bounds) == F + 1 else {})
    nnz_cap = int(kjt.values.numel() * self.capacity_factor) + 1024
    if W > 1:  # all ranks must agree on the layout
      import torch.distributed as dist
      t = torch.tensor([nnz_cap], device=dev, dtype=torch.int64)
      dist.all_reduce(t, op=dist.ReduceOp.MAX, group=m.group)
      nnz_cap = int(t.item())
    self.nnz_cap = nnz_cap
    # ---- pooled-buffer layout (identical on every rank) ----
    slot_off, off = {}, 0
    self.combine_descs = []
    for fname, col, width, L in self.layout:
      tp = m.plan.tables[m.feature_to_table[fname]]
      nslots = W if tp.placement is Placement.ROW_WISE else 1
      slot_off[fname] = off
      self.combine_descs.append(CombineDesc(off, nslots, tp.dim, col, L, self._rw_index_of(fname), 0))
      off += nslots * B * width
    pooled_elems = off
    # ---- gradient-buffer layout per destination rank ----
    # grad_off[r][fname]: element offset in rank r's gradient buffer of the [W*B, width_local] block
    self.grad_off = [dict() for _ in range(W)]
    grad_elems = [0] * W
    for fname, col, width, L in self.layout:
      tp = m.plan.tables[m.feature_to_table[fname]]
      for r in range(W):
        if tp.placement is Placement.TABLE_WISE and tp.owner != r:
          continue
        wl = width // W if tp.placement is Placement.COLUMN_WISE else width
        unit = tp.dim // W if tp.placement is Placement.COLUMN_WISE else tp.dim
        grad_elems[r] = (grad_elems[r] + unit - 1) // unit * unit   # block starts on a whole vector
        self.grad_off[r][fname] = grad_elems[r]
        grad_elems[r] += W * B * wl
    grad_cap = max(grad_elems)
    self.pooled_elems, self.grad_cap = pooled_elems, grad_cap
    self.buf = None
    # ---- per-stack work lists and occurrence storage ----
    self.slot_off = slot_off
    self.direct_ok = all(d.nslots == 1 for d in self.combine_descs) and all(
        m.plan.tables[m.feature_to_table[f]].dim % 8 == 0 for f, _, _, _ in self.layout)
    self.stacks = []
    for si, st in enumerate(m.plan.stacks):
      names = []
      for fname, col, width, L in self.layout:
        tp = m.plan.tables[m.feature_to_table[fname]]
        if tp.stack != si or (tp.placement is Placement.TABLE_WISE and tp.owner != m.rank):
          continue
        names.append(fname)
      info: dict[str, Any] = {"n_feats": len(names), "feat_names": names, "descs": {}}
      info["done"] = torch.zeros(4, dtype=torch.int32, device=dev)
      self.stacks.append(info)
    self.combine_dev = _device_struct_array(self.combine_descs, dev)
    push = []
    for fname, col, width, L in self.layout:
      tp = m.plan.tables[m.feature_to_table[fname]]
      d = PushGradDesc(KIND[tp.placement], tp.owner, tp.dim, col, L, self._rw_index_of(fname))
      for r in range(MAXW):
        d.grad_off[r] = self.grad_off[r].get(fname, -1) if r < W else -1
      push.append(d)
    self.push_dev = _device_struct_array(push, dev)
    self.done_ids = torch.zeros(4, dtype=torch.int32, device=dev)
    self.done_grads = torch.zeros(4, dtype=torch.int32, device=dev)
    self._occ_ready = False
    if W > 1 or not self.direct_ok:
      self._alloc_symm()

  def _alloc_symm(self):
    """One symmetric allocation holding flags, id copies, pooled slots and gradient blocks (the
    single-GPU direct path needs none of them, so it is only made when first required)."""
    if self.buf is not None:
      return
    m, W = self.m, self.m.world
    nnz_cap, pooled_elems, grad_cap = self.nnz_cap, self.pooled_elems, self.grad_cap
    cv = symm.Carver()
    n_chan = 2 + len(m.plan.stacks)
    self.flag_off = cv.take(n_chan * MAXW * 8)
    self.ids_off = [[(cv.take(nnz_cap * 4), cv.take(self.n_offsets * 4), cv.take(nnz_cap * 4))
                     for _ in range(W)] for _ in range(2)] if W > 1 else None
    self.pooled_off = [cv.take(pooled_elems * 2) for _ in range(2 if W > 1 else 1)]
    self.grad_buf_off = [cv.take(grad_cap * 2) for _ in range(2 if W > 1 else 1)]
    self.buf = symm.SymmBuffer(cv.off, m.group, m.device)

  def _rw_index_of(self, fname: str) -> int:
    """Position of `fname` among the row-sharded pooled features in feature order (what the bucketizing id push
    counts per owner), -1 for every other feature."""
    m = self.m
    seq_len = {f: L for f, _, _, L in self.layout}
    j = 0
    for f in m.feature_names:
      if m.plan.tables[m.feature_to_table[f]].placement is Placement.ROW_WISE and seq_len.get(f, 0) == 0:
        if f == fname:
          return j
        j += 1
    return -1

  def _bucket_state(self):
    """Device-side description of the features for the bucketizing id push, or None when it does not apply (a
    row-sharded pooled feature with a mean / sqrtn combiner needs the whole bag at the owner)."""
    if self._bucket is not None:
      return self._bucket or None
    m = self.m
    ok = self.bucketize and m.world > 1
    feats, n_rw = [], 0
    seq_len = {f: L for f, _, _, L in self.layout}
    for fname in m.feature_names:
      tp = m.plan.tables[m.feature_to_table[fname]]
      kind, rw_index = KIND.get(tp.placement, KIND[Placement.TABLE_WISE]), -1    # replicated: no rank is sent ids
      if tp.placement is Placement.ROW_WISE:
        if seq_len.get(fname, 0) > 0:
          kind = KIND[Placement.COLUMN_WISE]        # positions matter: every owner gets the whole sequence
        else:
          if m.config.specs[fname].combiner != "sum":
            ok = False
          rw_index, n_rw = n_rw, n_rw + 1
      feats.append(BucketFeat(kind, tp.owner if tp.placement is Placement.TABLE_WISE else -1, tp.rotation, rw_index))
    if not ok:
      self._bucket = False
      return None
    dev = m.device
    self._bucket = {"feats": _device_struct_array(feats, dev), "n_rw": n_rw,
                    "cnt": torch.zeros(max(n_rw, 1) * m.world * self.B, dtype=torch.int32, device=dev),
                    "tot": torch.zeros(max(n_rw, 1) * m.world, dtype=torch.int32, device=dev),
                    # per-owner id counts of every bag, one array per lookup that can be in flight: the combine of
                    # the forward and the gradient push of the backward skip the owners that got nothing of a bag
                    "raw": [torch.zeros(max(n_rw, 1) * m.world * self.B, dtype=torch.int32, device=dev)
                            for _ in range(max(self.pipeline_depth, 1))]}
    return self._bucket

  def partition_stats(self) -> dict[str, list[int]]:
    """Ids that the LAST bucketized batch of this rank sent to each owner, per row-sharded pooled feature
    (`{feature: [count for owner 0, owner 1, ...]}`; synchronises).  The maximum over owners and ranks is the
    `max_ids_per_partition` statistic of feedback-directed sizing (`id_pipeline.StatsRecorder`)."""
    b = self._bucket
    if not b or not b["n_rw"]:
      return {}
    m = self.m
    tot = b["tot"].reshape(b["n_rw"], m.world).cpu().tolist()
    seq_len = {f: L for f, _, _, L in self.layout}
    names = [f for f in m.feature_names
             if m.plan.tables[m.feature_to_table[f]].placement is Placement.ROW_WISE and seq_len.get(f, 0) == 0]
    return dict(zip(names, tot))

  def _need_mask(self) -> torch.Tensor:
    """uint8 per feature: bit r set when rank r holds rows (or columns) of the feature's table, i.e.
    needs its ids."""
    if self._need is None:
      m = self.m
      bits = []
      for fname in m.feature_names:
        tp = m.plan.tables[m.feature_to_table[fname]]
        bits.append(1 << tp.owner if tp.placement is Placement.TABLE_WISE else (1 << m.world) - 1)
      self._need = torch.tensor(bits, dtype=torch.uint8, device=m.device)
    return self._need

  def _feat_descs(self, si: int, direct: tuple[int, int] | None) -> torch.Tensor:
    """Device array of FeatDesc for stack `si`.  `direct=(ld, out_col)` makes the forward kernel
    store straight into a `[B, ld]` output matrix (and read gradients from a matrix of the same
    geometry); None uses the symmetric pooled / gradient buffers."""
    info = self.stacks[si]
    if direct not in info["descs"]:
      m = self.m
      feats = []
      tiles = 0
      for fname, col, width, L in self.layout:
        if fname not in info["feat_names"]:
          continue
        tp = m.plan.tables[m.feature_to_table[fname]]
        spec = m.config.specs[fname]
        if direct is not None:
          ld, out_col = direct
          slot, goff, stride = out_col + col, out_col + col, ld
        else:
          slot, goff, stride = self.slot_off[fname], self.grad_off[m.rank][fname], width
        # bags per warp of the tiled forward: a few hundred ids per tile whatever the bag size
        # (of a row-sharded feature a rank receives 1 / W of every bag when the senders bucketize the ids;
        # otherwise it scans all of them and gathers 1 / W: weigh the two)
        avg = self._avg_bag.get(fname, 1.0)
        if tp.placement is Placement.ROW_WISE and m.world > 1:
          sparse = self._bucket_state() is not None and L == 0
          avg = avg / m.world if sparse else (avg * 0.5 if m.world > 2 else avg)
        shift = 5 if avg <= 8 else 4 if avg <= 16 else 3 if avg <= 32 else 2 if avg <= 64 else 1
        bpt = 1 << shift
        feats.append(FeatDesc(m.feature_names.index(fname), KIND[tp.placement], tp.owner, tp.rotation,
                              tp.row_base, COMBINER[spec.combiner], tp.dim, tp.col_lo, slot, goff, L, stride, tp.vocab,
                              shift, tiles))
        tiles += m.world * ((self.B + bpt - 1) // bpt)
      info["descs"][direct] = _device_struct_array(feats, m.device)
      info["tiles"] = tiles
    return info["descs"][direct]

  def _ensure_occ(self, kjt):
    """Occurrence / sort / scratch storage (training only), sized from the batch."""
    if self._occ_ready:
      return
    m, dev, W, B = self.m, self.m.device, self.m.world, self.B
    per_feat = {}
    off = kjt.offsets
    for fi, fname in enumerate(m.feature_names):
      per_feat[fname] = int(off[(fi + 1) * B].item() - off[fi * B].item())
    for si, info in enumerate(self.stacks):
      cap = 0
      for fname in info["feat_names"]:
        tp = m.plan.tables[m.feature_to_table[fname]]
        n = per_feat[fname] * W
        if tp.placement is Placement.ROW_WISE and W > 1:
          n = int(n / W * 1.5) + 4096   # MOD sharding spreads ids evenly; 50 % head-room
        cap += n
      cap = int(cap * self.capacity_factor) + 1024
      info["occ_cap"] = cap
      # one occurrence list per lookup that can be in flight; `sorted` says which of the two (keys, vals)
      # buffers of a set holds the sorted list
      info["sets"] = [dict(keys=torch.empty(2, cap, dtype=torch.int32, device=dev),
                           vals=torch.empty(2, cap, dtype=torch.int32, device=dev),
                           gain=torch.empty(cap, 2, dtype=torch.float32, device=dev) if self.has_gains else None,
                           count=torch.zeros(1, dtype=torch.int32, device=dev), sorted=0)
                      for _ in range(self.pipeline_depth)]
      dloc = m.plan.stacks[si].dim
      info["scratch"] = torch.zeros((cap + 127) // 128, dloc, dtype=torch.float32, device=dev)
      words = int(self.lib.recml_radix_sort_scratch_words(c_ll(cap)))
      info["sort_scratch"] = torch.empty(words, dtype=torch.int32, device=dev)
      info["key_bits"] = max(1, int(max(m.plan.stacks[si].rows, 1) - 1).bit_length())
    self._occ_ready = True
    self._push_hyper()

  def _flag_ptr(self, rank: int, chan: int, src: int) -> int:
    if self.buf is None:
      return 0
    return self.buf.peer_ptr(rank, self.flag_off + (chan * MAXW + src) * 8)

  # -- forward ---------------------------------------------------------------------------------------------
  def forward(self, kjt: jagged_lib.KeyedJagged, training: bool, out: torch.Tensor | None = None,
              out_col: int = 0):
    m = self.m
    W, dev = m.world, m.device
    if self.B is None:
      self._setup(kjt)
    if kjt.batch_size() != self.B:
      raise ValueError(f"fused backend was set up for batch {self.B}, got {kjt.batch_size()}")
    streams.join("emb_bwd", "emb_sort", device=dev)    # the previous step's table update comes first
    if W > 1 and kjt.values.numel() > self.nnz_cap:      # the exchange buffers of the peers are sized for this
      raise ValueError(f"batch has {kjt.values.numel()} ids, the id exchange buffers hold {self.nnz_cap}")
    assert kjt.values.dtype == torch.int32 and kjt.offsets.dtype == torch.int32
    if training:
      self._ensure_occ(kjt)
    # The step's sequence number lives on the device (ticked here, read by every kernel of the step),
    # so a captured CUDA graph advances it on every replay; `self.seq` mirrors it for buffer parity.
    self.seq += 1
    par = (self.seq & 1) if W > 1 else 0
    st = _lib.stream()
    _lib.check_rc(self.lib.recml_tick(_lib.ptr(self.seq_dev), st), "tick")
    seq = SeqRef(self.seq_dev.data_ptr(), 1, 0, 0) if self.pipeline_depth == 1 else SeqRef(None, 0, 0, self.seq)
    oset = 0
    if training:
      oset = self._train_calls % self.pipeline_depth
      self._train_calls += 1
    gains = self.has_gains
    B = self.B
    if out is None:
      out = _lib.debug_empty((B, self.width), torch.bfloat16, dev, "pooled embedding output")
      out_col = 0
    assert out.dtype == torch.bfloat16 and out.stride(1) == 1
    direct = None
    if self.direct_ok and W == 1 and out.stride(0) % 8 == 0 and out_col % 8 == 0 and out.data_ptr() % 16 == 0:
      direct = (out.stride(0), out_col)
    if direct is None:
      self._alloc_symm()
    ids = IdPtrs()
    bucket = self._bucket_state() if W > 1 else None
    if bucket is not None:
      p = BucketizeParams()
      p.values, p.offsets = kjt.values.data_ptr(), kjt.offsets.data_ptr()
      p.weights = kjt.weights.data_ptr() if kjt.weights is not None else None
      p.n_feats, p.B, p.W, p.me, p.n_rw = len(m.feature_names), B, W, m.rank, bucket["n_rw"]
      p.feats, p.cnt, p.tot = bucket["feats"].data_ptr(), bucket["cnt"].data_ptr(), bucket["tot"].data_ptr()
      if len(bucket["raw"]) < self.pipeline_depth:      # the depth was raised after the first lookup
        bucket["raw"] += [torch.zeros_like(bucket["raw"][0]) for _ in range(self.pipeline_depth - len(bucket["raw"]))]
      p.cnt_raw = bucket["raw"][oset % len(bucket["raw"])].data_ptr()
      vo, oo, wo = self.ids_off[par][m.rank]
      for r in range(W):
        p.dst_values[r] = self.buf.peer_ptr(r, vo)
        p.dst_offsets[r] = self.buf.peer_ptr(r, oo)
        p.dst_weights[r] = self.buf.peer_ptr(r, wo)
        p.flags[r] = self._flag_ptr(r, 0, m.rank)
      p.done_counter, p.seq = self.done_ids.data_ptr(), seq
      _lib.check_rc(self.lib.recml_emb_bucketize_push(ctypes.byref(p), st), "emb_bucketize_push")
      _lib.LAUNCHES["count"] += 2 if bucket["n_rw"] else 0
      for s in range(W):
        vo, oo, wo = self.ids_off[par][s]
        ids.values[s] = self.buf.peer_ptr(m.rank, vo)
        ids.offsets[s] = self.buf.peer_ptr(m.rank, oo)
        ids.weights[s] = self.buf.peer_ptr(m.rank, wo) if kjt.weights is not None else None
    elif W > 1:
      p = PushIdsParams()
      p.values, p.offsets = kjt.values.data_ptr(), kjt.offsets.data_ptr()
      p.weights = kjt.weights.data_ptr() if kjt.weights is not None else None
      p.nnz, p.n_offsets, p.W, p.me = kjt.values.numel(), self.n_offsets, W, m.rank
      vo, oo, wo = self.ids_off[par][m.rank]
      for r in range(W):
        p.dst_values[r] = self.buf.peer_ptr(r, vo)
        p.dst_offsets[r] = self.buf.peer_ptr(r, oo)
        p.dst_weights[r] = self.buf.peer_ptr(r, wo)
        p.flags[r] = self._flag_ptr(r, 0, m.rank)
      p.done_counter, p.seq = self.done_ids.data_ptr(), seq
      p.need, p.n_feats, p.B = self._need_mask().data_ptr(), len(m.feature_names), B
      _lib.check_rc(self.lib.recml_emb_push_ids(ctypes.byref(p), st), "emb_push_ids")
      for s in range(W):
        vo, oo, wo = self.ids_off[par][s]
        ids.values[s] = self.buf.peer_ptr(m.rank, vo)
        ids.offsets[s] = self.buf.peer_ptr(m.rank, oo)
        ids.weights[s] = self.buf.peer_ptr(m.rank, wo) if kjt.weights is not None else None
    else:
      ids.values[0], ids.offsets[0] = kjt.values.data_ptr(), kjt.offsets.data_ptr()
      ids.weights[0] = kjt.weights.data_ptr() if kjt.weights is not None else None
    for si, info in enumerate(self.stacks):
      occ = info["sets"][oset] if training else None
      if training:
        occ["count"].zero_()
      fp = FwdParams()
      fp.ids = ids
      fp.feats, fp.n_feats = self._feat_descs(si, direct).data_ptr(), info["n_feats"]
      fp.W, fp.me, fp.B, fp.dloc = W, m.rank, B, m.plan.stacks[si].dim
      fp.table = m.stack_weights[si].data_ptr()
      for r in range(W):
        fp.pooled[r] = out.data_ptr() if direct is not None else self.buf.peer_ptr(r, self.pooled_off[par])
        fp.flags[r] = self._flag_ptr(r, 1 + si, m.rank)
      fp.grad_ld = direct[0] if direct is not None else 0
      if training:
        fp.occ_key, fp.occ_val = occ["keys"][0].data_ptr(), occ["vals"][0].data_ptr()
        fp.occ_gain = occ["gain"].data_ptr() if gains else None
        fp.occ_count, fp.occ_cap = occ["count"].data_ptr(), info["occ_cap"]
        fp.dropped = self.dropped.data_ptr() if self.dropped is not None else None
      fp.wait_flags = self._flag_ptr(m.rank, 0, 0) if W > 1 else None
      fp.prefetch = self.fwd_prefetch
      fp.tiled = int(self.fwd_tiled and all(L == 0 for f_, _, _, L in self.layout if f_ in info["feat_names"]))
      fp.total_tiles = info.get("tiles", 0)
      fp.prefiltered = int(bucket is not None)
      fp.done_counter, fp.seq, fp.status = info["done"].data_ptr(), seq, self.status.data_ptr()
      if info["n_feats"] or W > 1:
        _lib.check_rc(self.lib.recml_emb_fwd(ctypes.byref(fp), c_int(int(training)), c_int(int(gains)), st),
                      "emb_fwd")
    if training:
      self._sort_occurrences(oset)
    odt = m.config.output_dtype or torch.bfloat16
    if direct is not None:
      res = out[:, out_col:out_col + self.width]
      res = res if odt == torch.bfloat16 else res.to(odt)
      return res, ({"seq": seq, "par": par, "kjt": kjt, "direct": direct, "set": oset} if training else None)
    cp = CombineParams()
    cp.pooled = self.buf.peer_ptr(m.rank, self.pooled_off[par])
    cp.feats, cp.n_feats, cp.B = self.combine_dev.data_ptr(), len(self.combine_descs), B
    cp.out, cp.ld_out = out.data_ptr() + out_col * 2, out.stride(0)
    # wait on the pooled channels of every stack: channels 1..n_stacks are contiguous
    cp.wait_flags = self._flag_ptr(m.rank, 1, 0) if W > 1 else None
    cp.W, cp.n_chan, cp.seq, cp.status = W, len(self.stacks), seq, self.status.data_ptr()
    cp.cnt_raw = bucket["raw"][oset % len(bucket["raw"])].data_ptr() if bucket is not None else None
    _lib.check_rc(self.lib.recml_emb_combine(ctypes.byref(cp), st), "emb_combine")
    res = out[:, out_col:out_col + self.width]
    res = res if odt == torch.bfloat16 else res.to(odt)
    saved = {"seq": seq, "par": par, "kjt": kjt, "direct": None, "set": oset} if training else None
    return res, saved

  def _sort_occurrences(self, oset: int = 0) -> None:
    """Groups the step's occurrence list by row.  The list is complete once the forward kernels have run
    and nothing else of the forward pass needs the result, so the sort goes to a side stream and runs
    beside the dense forward; the backward waits for it."""
    use_side = self.side_streams
    s = streams.fork("emb_sort", self.m.device) if use_side else torch.cuda.current_stream(self.m.device)
    with torch.cuda.stream(s):
      st = _lib.stream()
      for info in self.stacks:
        n = info["occ_cap"]
        if n <= 0 or info["n_feats"] == 0:
          continue
        occ = info["sets"][oset]
        rc = self.lib.recml_radix_sort_pairs(
            _lib.ptr(occ["keys"][0]), _lib.ptr(occ["vals"][0]), _lib.ptr(occ["keys"][1]),
            _lib.ptr(occ["vals"][1]), _lib.ptr(occ["count"]), c_ll(n), c_int(info["key_bits"]),
            _lib.ptr(info["sort_scratch"]), _lib.ptr(self.status), st)
        if rc < 0:
          raise _lib.NativeError(f"radix sort failed with code {rc}")
        _lib.LAUNCHES["count"] += 4 * ((info["key_bits"] + 8) // 9) - 1    # four kernels per pass
        occ["sorted"] = rc

  # -- backward ----------------------------------------------------------------------------------------------
  @torch.no_grad()
  def backward(self, saved: Any, grad_out: torch.Tensor) -> None:
    """Launches the gradient push and the table update.  With side streams on, they are issued on the
    "emb_bwd" stream (after everything issued so far on the current stream and after the sort), so the
    caller's stream is free to go on with work that does not touch the tables; `streams.join("emb_bwd")`
    (done by the next forward and by `State.update`) orders later work behind the update."""
    m = self.m
    if grad_out.dtype != torch.bfloat16:
      grad_out = grad_out.to(torch.bfloat16)
    if grad_out.stride(-1) != 1:
      grad_out = grad_out.contiguous()
    from recml_b200.utils import graphs
    if not graphs.capturing():
      self._push_hyper()
    if not self.side_streams:
      self._backward_on_current(saved, grad_out)
      return
    s = streams.fork("emb_bwd", m.device)
    streams.chain("emb_bwd", "emb_sort", m.device)
    streams.keep_alive_on(s, grad_out)
    with torch.cuda.stream(s):
      self._backward_on_current(saved, grad_out)

  def _backward_on_current(self, saved: Any, grad_out: torch.Tensor) -> None:
    m = self.m
    W, B = m.world, self.B
    st = _lib.stream()
    seq, par = saved["seq"], saved["par"]
    direct = saved["direct"]
    gchan = 1 + len(self.stacks)
    if direct is not None:
      ld, out_col = direct
      base = grad_out.data_ptr() - out_col * 2
      if grad_out.stride(0) != ld or base % 16:
        full = torch.empty(B, ld, dtype=torch.bfloat16, device=grad_out.device)
        full[:, out_col:out_col + self.width] = grad_out
        base, saved["_keep"] = full.data_ptr(), full
      grads_ptr, val_scale = base, 8
    else:
      pg = PushGradParams()
      pg.grad, pg.ld = grad_out.data_ptr(), grad_out.stride(0)
      pg.feats, pg.n_feats, pg.B, pg.W, pg.me = self.push_dev.data_ptr(), len(self.layout), B, W, m.rank
      for r in range(W):
        pg.dst[r] = self.buf.peer_ptr(r, self.grad_buf_off[par])
        pg.flags[r] = self._flag_ptr(r, gchan, m.rank)
      pg.done_counter, pg.seq = self.done_grads.data_ptr(), seq
      bucket = self._bucket if isinstance(self._bucket, dict) else None
      pg.cnt_raw = bucket["raw"][saved.get("set", 0) % len(bucket["raw"])].data_ptr() if bucket is not None else None
      _lib.check_rc(self.lib.recml_emb_push_grads(ctypes.byref(pg), st), "emb_push_grads")
      grads_ptr, val_scale = self.buf.peer_ptr(m.rank, self.grad_buf_off[par]), None
    for si, info in enumerate(self.stacks):
      # The occurrence count stays on the device: every kernel reads it there, so backward never
      # synchronises with the host.
      n = info["occ_cap"]
      opt = m.plan.stacks[si].optimizer
      occ = info["sets"][saved.get("set", 0)]
      srt = occ["sorted"]
      bp = BwdParams()
      bp.keys, bp.vals = occ["keys"][srt].data_ptr(), occ["vals"][srt].data_ptr()
      bp.occ_gain = occ["gain"].data_ptr() if self.has_gains else None
      bp.n_occ = occ["count"].data_ptr()
      bp.grads = grads_ptr
      bp.val_scale = val_scale if val_scale is not None else m.plan.stacks[si].dim
      bp.table = m.stack_weights[si].data_ptr()
      names = opt.slot_names()
      slots = m.stack_slots[si]
      bp.slot0 = slots[names[0]].data_ptr() if len(names) > 0 else None
      bp.slot1 = slots[names[1]].data_ptr() if len(names) > 1 else None
      bp.dloc, bp.opt = m.plan.stacks[si].dim, OPT[opt.kind]
      hp = opt.hyperparams(m.step_count)
      for i in range(6):
        bp.hp[i] = hp[i] if i < len(hp) else 0.0
      bp.grad_scale = m.grad_scale
      bp.scratch = info["scratch"].data_ptr()
      bp.wait_flags = self._flag_ptr(m.rank, gchan, 0) if (W > 1 and direct is None) else None
      bp.W, bp.seq, bp.status = W, seq, self.status.data_ptr()
      bp.hp_dev = self._hp_dev[si].data_ptr()
      bp.n_cap = n
      if n > 0 or W > 1:
        _lib.check_rc(self.lib.recml_emb_bwd_update(ctypes.byref(bp), c_ll(max(n, 1)), c_int(int(self.has_gains)),
                                                    c_int(self.bwd_blocks_per_sm), st), "emb_bwd_update")
