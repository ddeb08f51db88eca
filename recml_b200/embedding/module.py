"""`ShardedEmbedding`: the GPU sharded-embedding layer.

Role of the reference's `SparsecoreEmbed` + `sparsecore_lookup`
(`recml/layers/linen/sparsecore.py:357-444`, `recml/core/ops/embedding_ops.py:47-110`):
forward = gather rows, pool every bag, return batch-sharded activations; backward =
route the activation gradients to the owners, aggregate per unique row and APPLY the
table optimizer there (the tables never appear in the dense optimizer).

Two interchangeable backends share the plan, the storage and the semantics:
  * "fused"      — sm_100a kernels over NVLink peer memory (`recml_b200.embedding.fused`)
  * "collective" — torch ops + `torch.distributed` collectives (gloo on CPU, NCCL as the
                   stand-in baseline on GPU); also the oracle in tests.
"""
from __future__ import annotations

import os

import dataclasses
import math
from typing import Any, Callable, Mapping, Sequence

import torch
import torch.distributed as dist
from torch import nn

from recml_b200.ckpt.manager import ShardedLeaf
from recml_b200.embedding import jagged as jagged_lib
from recml_b200.embedding import planner as planner_lib
from recml_b200.embedding import specs as specs_lib
from recml_b200.embedding.planner import Placement


@dataclasses.dataclass
class ShardedEmbeddingConfig:
  """Counterpart of `SparsecoreConfig` (`sparsecore.py:94-269`)."""
  specs: Mapping[str, specs_lib.EmbeddingSpec]
  optimizer: specs_lib.OptimizerSpec
  sharding_strategy: str = "auto"          # "auto" | "MOD" (all row-wise) | "table" | "column"
  placement_overrides: Mapping[str, Placement] | None = None
  row_wise_min_bytes: int | None = None   # None: cost-balanced placement (see planner)
  replicate_max_rows: int = 0
  allow_id_dropping: bool = False
  ids_per_sample: Mapping[str, float] | None = None
  # per FEATURE: share of its ids on the most frequent row, or the shares of rows 0, 1, 2, ... (planner)
  hot_row_share: Mapping[str, Any] | None = None
  # per FEATURE: (ids per sample by residue class id % world, distinct ids per sample by class), e.g. from
  # `embedding.stats.batch_residue_stats` on the first batch; the planner's most precise cost input
  residue_stats: Mapping[str, Any] | None = None
  backend: str = "auto"                    # "auto" | "fused" | "collective"
  output_dtype: torch.dtype | None = None
  seed: int = 0

  def table_specs(self) -> tuple[list[specs_lib.TableSpec], dict[str, str]]:
    """Tables (deduplicated by `table_name`) and feature→table mapping."""
    tables: dict[str, specs_lib.TableSpec] = {}
    feature_to_table = {}
    for fname, s in self.specs.items():
      tname = s.table_name or fname
      if tname in tables:
        t = tables[tname]
        if (t.vocabulary_size, t.embedding_dim) != (s.input_dim, s.embedding_dim):
          raise ValueError(f"Features sharing table {tname!r} disagree on its shape.")
      else:
        tables[tname] = specs_lib.TableSpec(
            tname, s.input_dim, s.embedding_dim, s.optimizer or self.optimizer, s.combiner,
            s.initializer)
      feature_to_table[fname] = tname
    return list(tables.values()), feature_to_table


def _world_rank(group) -> tuple[int, int]:
  if dist.is_available() and dist.is_initialized():
    return dist.get_world_size(group), dist.get_rank(group)
  return 1, 0


class _LookupFn(torch.autograd.Function):
  """Forward returns pooled activations; backward applies the table optimizer."""

  @staticmethod
  def forward(ctx, anchor, module, kjt, training, out, out_col):
    ctx.module = module
    if out is not None:
      res, saved = module._backend.forward(kjt, training=training, out=out, out_col=out_col)
    else:
      res, saved = module._backend.forward(kjt, training=training)
    out = res
    ctx.saved = saved
    return out

  @staticmethod
  def backward(ctx, grad_out):
    if ctx.saved is not None:
      ctx.module._backend.backward(ctx.saved, grad_out)
      ctx.module.step_count += 1
    return torch.zeros_like(ctx.module.anchor), None, None, None, None, None


class ShardedEmbedding(nn.Module):
  """Holds this rank's shards of every table and performs the sharded lookup.

  `forward(kjt)` takes a `KeyedJagged` with this rank's batch and returns
  `[B_local, F, D]` when all features share D, else a dict name → `[B_local, D_f]`;
  sequence features (`max_sequence_length` set) come back as `[B_local, L, D]` in
  the dict form.  Calling `.backward()` through the output updates the tables.
  """

  def __init__(self, config: ShardedEmbeddingConfig, *, device: torch.device | str | None = None,
               group=None):
    super().__init__()
    self.config = config
    self.group = group
    self.world, self.rank = _world_rank(group)
    self.device = torch.device(device) if device is not None else (
        torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
        else torch.device("cpu"))
    tables, self.feature_to_table = config.table_specs()
    self.table_specs = {t.name: t for t in tables}
    self.feature_names = tuple(config.specs)
    overrides = dict(config.placement_overrides or {})
    default = {"MOD": Placement.ROW_WISE, "table": Placement.TABLE_WISE,
               "column": Placement.COLUMN_WISE}.get(config.sharding_strategy)
    ids = dict(config.ids_per_sample or {})
    table_ids = {}
    for f, t in self.feature_to_table.items():
      table_ids[t] = table_ids.get(t, 0.0) + ids.get(f, 1.0)
    hot: dict[str, list] = {}      # per table: ids-weighted mean of its features' share lists
    wsum: dict[str, float] = {}
    for f, share in (config.hot_row_share or {}).items():
      t = self.feature_to_table[f]
      w = ids.get(f, 1.0)
      lst = [float(share)] if isinstance(share, (int, float)) else [float(x) for x in share]
      acc = hot.setdefault(t, [])
      for k, x in enumerate(lst):
        if k >= len(acc):
          acc.append(0.0)
        acc[k] += x * w
      wsum[t] = wsum.get(t, 0.0) + w
    res: dict[str, list] = {}      # per table: sums over its features; distinct ids capped by the rows of a class
    for f, (occ, uniq) in (config.residue_stats or {}).items():
      if len(occ) != self.world:
        continue
      t = self.feature_to_table[f]
      acc = res.setdefault(t, [[0.0] * self.world, [0.0] * self.world])
      for q in range(self.world):
        acc[0][q] += float(occ[q])
        acc[1][q] += float(uniq[q])
    self.plan = planner_lib.plan_tables(
        tables, self.world, self.rank, ids_per_sample=table_ids, residue_stats=res,
        imbalance_tolerance=float(os.environ.get("RECML_PLAN_TOLERANCE", "0.15")),
        hot_row_share={t: [x / max(wsum[t], 1e-9) for x in acc] for t, acc in hot.items()},
        row_wise_min_bytes=config.row_wise_min_bytes,
        replicate_max_rows=config.replicate_max_rows, overrides=overrides, default=default)
    # Storage: one weight buffer per stack (+ optimizer slots), tagged so the dense
    # optimizer / gradient all-reduce skip them.
    self.stack_weights: list[torch.Tensor] = []
    self.stack_slots: list[dict[str, torch.Tensor]] = []
    for si, st in enumerate(self.plan.stacks):
      w = torch.empty(max(st.rows, 1), st.dim, dtype=torch.float32, device=self.device)
      w._recml_sharded = True
      self.register_buffer(f"stack_{si}_table", w, persistent=False)
      self.stack_weights.append(w)
      slots = {}
      for s in st.optimizer.slot_names():
        shape = (max(st.rows, 1),) if st.optimizer.slot_is_rowwise(s) else (max(st.rows, 1), st.dim)
        t = torch.full(shape, st.optimizer.slot_init(s), dtype=torch.float32, device=self.device)
        t._recml_sharded = True
        self.register_buffer(f"stack_{si}_{s}", t, persistent=False)
        slots[s] = t
      self.stack_slots.append(slots)
    # Replicated small tables are ordinary parameters trained by the dense optimizer.
    self.replicated = nn.ParameterDict()
    for t in tables:
      if self.plan.tables[t.name].placement is Placement.REPLICATED:
        self.replicated[t.name] = nn.Parameter(
            torch.empty(t.vocabulary_size, t.embedding_dim, device=self.device))
    # The anchor gives autograd a differentiable input so backward always runs.
    self.anchor = nn.Parameter(torch.zeros((), device=self.device))
    self.anchor._recml_sharded = True
    self.step_count = 0
    # Activation gradients arrive from `world` data-parallel ranks; like dense gradients they are
    # averaged (each rank scales its loss by 1/local_batch), so the summed row gradient is divided
    # by the world size before the row optimizer sees it.
    self.grad_scale = 1.0 / self.world
    self.reset_parameters()
    self._backend = self._make_backend(config.backend)

  # -- initialisation: every row is generated from (seed, table, global row) so the
  #    values do not depend on the world size or placement --------------------------------
  def _default_init(self, spec: specs_lib.TableSpec):
    if spec.initializer is not None:
      return spec.initializer
    return specs_lib.truncated_normal_init(1.0 / math.sqrt(spec.embedding_dim))

  @torch.no_grad()
  def reset_parameters(self, chunk_rows: int = 1 << 22):
    for ti, (name, tp) in enumerate(self.plan.tables.items()):
      spec = self.table_specs[name]
      init = self._default_init(spec)
      if tp.placement is Placement.REPLICATED:
        gen = torch.Generator(device=self.device).manual_seed(self.config.seed * 1000003 + ti)
        init(self.replicated[name].data, gen)
        continue
      if tp.local_rows == 0:
        continue
      dst = self.stack_weights[tp.stack][tp.row_base:tp.row_base + tp.local_rows]
      if tp.vocab * tp.dim <= (1 << 24):
        # small table: build the full table deterministically, then cut this rank's part
        gen = torch.Generator(device="cpu").manual_seed(self.config.seed * 1000003 + ti)
        full = torch.empty(tp.vocab, tp.dim)
        init(full, gen)
        dst.copy_(self._cut(full, tp))
      else:
        # large table: per-rank seeded on-device init in chunks (never materialised whole)
        gen = torch.Generator(device=self.device).manual_seed(
            (self.config.seed * 1000003 + ti) * 4099 + self.rank)
        for a in range(0, tp.local_rows, chunk_rows):
          init(dst[a:a + chunk_rows], gen)

  def _cut(self, full: torch.Tensor, tp: planner_lib.TablePlan) -> torch.Tensor:
    if tp.placement is Placement.ROW_WISE:
      res = (self.rank - tp.rotation) % self.world
      return full[res::self.world]
    if tp.placement is Placement.COLUMN_WISE:
      return full[:, tp.col_lo:tp.col_lo + tp.local_dim]
    return full

  def _make_backend(self, name: str):
    if name == "auto":
      name = "fused" if self.device.type == "cuda" else "collective"
    if name == "fused":
      from recml_b200.embedding import fused
      return fused.FusedBackend(self)
    from recml_b200.embedding import collective
    return collective.CollectiveBackend(self)

  # -- forward -------------------------------------------------------------------------------
  def forward(self, kjt: jagged_lib.KeyedJagged, *, flat: bool = False, out: torch.Tensor | None = None,
              out_col: int = 0) -> Any:
    """`flat=True` returns the `[B, ΣD]` concatenation of the sharded features in feature
    order (what DLRM consumes); otherwise `[B, F, D]` when every feature is pooled with
    the same D, else a dict feature → `[B, D]` / `[B, L, D]`."""
    if tuple(kjt.keys) != self.feature_names:
      raise ValueError(f"Expected features {self.feature_names}, got {kjt.keys}")
    out = _LookupFn.apply(self.anchor, self, kjt, torch.is_grad_enabled() and self.training,
                          out if flat else None, out_col)
    from recml_b200.embedding import collective
    layout, _ = collective.feature_layout(self)
    has_rep = len(layout) != len(self.feature_names)
    if flat and not has_rep:
      return out
    d = self.uniform_dim()
    if (not has_rep and not flat and d is not None and all(L == 0 for _, _, _, L in layout)
        and out.is_contiguous() and out.shape[1] == len(layout) * d):
      return out.view(out.shape[0], len(layout), d)      # a view: nothing is copied, forward or backward
    feats = {}
    # one split (whose backward is one concatenation) instead of a slice per feature, whose backward
    # would allocate and add a full-width gradient per feature
    contiguous_cols = all(col == sum(w for _, _, w, _ in layout[:i]) for i, (_, col, _, _) in enumerate(layout))
    pieces = (torch.split(out, [w for _, _, w, _ in layout], dim=1) if contiguous_cols and
              sum(w for _, _, w, _ in layout) == out.shape[1] else [out[:, c:c + w] for _, c, w, _ in layout])
    for (f, col, width, L), x in zip(layout, pieces):
      D = self.config.specs[f].embedding_dim
      feats[f] = x.reshape(x.shape[0], L, D) if L else x
    for f in self.feature_names:
      if f not in feats:
        feats[f] = self._replicated_lookup(kjt, f).to(out.dtype)
    if flat:
      return torch.cat([feats[f].reshape(feats[f].shape[0], -1) for f in self.feature_names], dim=1)
    if d is not None:
      return torch.stack([feats[f] for f in self.feature_names], dim=1)
    return feats

  def _replicated_lookup(self, kjt: jagged_lib.KeyedJagged, fname: str) -> torch.Tensor:
    """Small replicated tables: differentiable torch lookup on the local batch only."""
    from recml_b200.embedding import collective
    spec = self.config.specs[fname]
    table = self.replicated[self.feature_to_table[fname]]
    vals, offs, w = kjt.feature(fname)
    B = offs.numel() - 1
    lens = offs[1:] - offs[:-1]
    bag = torch.repeat_interleave(torch.arange(B, device=vals.device), lens)
    gains = collective.bag_gains(spec, lens, bag, w)
    rows = table[vals.long()] * gains[:, None]
    if spec.max_sequence_length:
      L = spec.max_sequence_length
      pos = torch.arange(vals.numel(), device=vals.device) - offs[:-1][bag]
      keep = pos < L
      out = rows.new_zeros(B * L, table.shape[1])
      return out.index_add(0, (bag * L + pos)[keep], rows[keep]).view(B, L, -1)
    return rows.new_zeros(B, table.shape[1]).index_add(0, bag, rows)

  def uniform_dim(self) -> int | None:
    dims = {s.embedding_dim for s in self.config.specs.values()}
    seq = any(s.max_sequence_length is not None for s in self.config.specs.values())
    return dims.pop() if len(dims) == 1 and not seq else None

  # -- table access (API of `gather_table` / `fetch_tables`, `sparsecore.py:447-549`) ------------
  @torch.no_grad()
  def gather_table(self, name: str, slot: str | None = None) -> torch.Tensor:
    """The full un-sharded `[vocab, dim]` table (or optimizer slot) on every rank."""
    tp = self.plan.tables[name]
    if tp.placement is Placement.REPLICATED:
      return self.replicated[name].detach().clone()
    src = self.stack_weights[tp.stack] if slot is None else self.stack_slots[tp.stack][slot]
    local = src[tp.row_base:tp.row_base + tp.local_rows]
    rowwise_slot = local.ndim == 1
    if rowwise_slot:
      local = local[:, None]
    if self.world == 1:
      out = local.clone()
    elif tp.placement is Placement.TABLE_WISE:
      out = torch.empty(tp.vocab, local.shape[1], device=self.device)
      if self.rank == tp.owner:
        out.copy_(local)
      dist.broadcast(out, src=dist.get_global_rank(self.group, tp.owner) if self.group else tp.owner,
                     group=self.group)
    else:
      rows_max = (tp.vocab + self.world - 1) // self.world if tp.placement is Placement.ROW_WISE \
          else tp.vocab
      pad = torch.zeros(rows_max, local.shape[1], device=self.device)
      pad[:local.shape[0]] = local
      parts = [torch.empty_like(pad) for _ in range(self.world)]
      dist.all_gather(parts, pad, group=self.group)
      if tp.placement is Placement.ROW_WISE:
        out = torch.empty(tp.vocab, local.shape[1], device=self.device)
        for r in range(self.world):
          res = (r - tp.rotation) % self.world
          n = planner_lib._local_rows(tp.vocab, self.world, r, tp.rotation)
          out[res::self.world] = parts[r][:n]
      elif rowwise_slot:
        out = parts[0]
      else:
        out = torch.cat(parts, dim=1)
    return out[:, 0] if rowwise_slot else out

  def fetch_tables(self) -> dict[str, torch.Tensor]:
    """All tables, un-sharded, on the host."""
    return {n: self.gather_table(n).cpu() for n in self.plan.tables}

  @torch.no_grad()
  def load_table(self, name: str, full: torch.Tensor, slot: str | None = None) -> None:
    tp = self.plan.tables[name]
    if tp.placement is Placement.REPLICATED:
      self.replicated[name].data.copy_(full)
      return
    if tp.local_rows == 0:
      return
    dst = (self.stack_weights[tp.stack] if slot is None else self.stack_slots[tp.stack][slot])
    dst = dst[tp.row_base:tp.row_base + tp.local_rows]
    if dst.ndim == 1:
      piece = full if tp.placement is not Placement.ROW_WISE else \
          full[(self.rank - tp.rotation) % self.world::self.world]
      dst.copy_(piece.to(self.device))
    else:
      dst.copy_(self._cut(full, tp).to(self.device))

  # -- checkpointing: each table is ONE global array, chunked by its shards ----------------------
  def sharded_state_dict(self) -> dict[str, Any]:
    out: dict[str, Any] = {"step": torch.tensor(self.step_count, dtype=torch.int64)}
    for name, tp in self.plan.tables.items():
      if tp.placement is Placement.REPLICATED:
        continue
      entry = {"table": self._leaf(tp, self.stack_weights[tp.stack])}
      for s, buf in self.stack_slots[tp.stack].items():
        entry[s] = self._leaf(tp, buf)
      out[name] = entry
    return out

  def _leaf(self, tp: planner_lib.TablePlan, buf: torch.Tensor) -> ShardedLeaf:
    local = buf[tp.row_base:tp.row_base + tp.local_rows]
    rowwise = local.ndim == 1
    W = self.world
    if tp.placement is Placement.ROW_WISE:
      # stored in MOD layout: global array [W, ceil(V/W)(, D)], block r = residue r's rows
      rows = (tp.vocab + W - 1) // W
      res = (self.rank - tp.rotation) % W
      gshape = (W, rows) if rowwise else (W, rows, tp.dim)
      chunk = (1, rows) if rowwise else (1, rows, tp.dim)
      idx = (res, 0) if rowwise else (res, 0, 0)
      return ShardedLeaf(local[None], gshape, idx, chunk, mod={"vocab": tp.vocab, "world": W})
    if tp.placement is Placement.COLUMN_WISE:
      if rowwise:
        return ShardedLeaf(local, (tp.vocab,), (0,), (tp.vocab,), write=self.rank == 0)
      return ShardedLeaf(local, (tp.vocab, tp.dim), (0, self.rank), (tp.vocab, tp.local_dim))
    gshape = (tp.vocab,) if rowwise else (tp.vocab, tp.dim)
    if self.rank == tp.owner:
      return ShardedLeaf(local, gshape, (0,) * len(gshape), gshape)
    return ShardedLeaf(local.new_zeros((0,) + gshape[1:]), gshape, (0,) * len(gshape), gshape,
                       write=False)

  @torch.no_grad()
  def load_sharded_state_dict(self, sd: Mapping[str, Any]) -> None:
    self.step_count = int(sd["step"])
    for name, tp in self.plan.tables.items():
      if tp.placement is Placement.REPLICATED or tp.local_rows == 0:
        continue
      for key, buf in [("table", self.stack_weights[tp.stack])] + list(
          self.stack_slots[tp.stack].items()):
        if key not in sd[name]:          # an export without optimizer slots: keep the initial ones
          continue
        dst = buf[tp.row_base:tp.row_base + tp.local_rows]
        src = torch.as_tensor(sd[name][key])
        if tp.placement is Placement.ROW_WISE:
          src = src[0][:tp.local_rows]
        dst.copy_(src.to(self.device))


def cpu_lookup(config: ShardedEmbeddingConfig, tables: Mapping[str, torch.Tensor],
               inputs: jagged_lib.KeyedJagged) -> dict[str, torch.Tensor]:
  """Host oracle (`sparsecore.py:552-625`, with all three combiners working, weighted or
  not).  `tables` maps TABLE name → full `[V, D]` tensor."""
  out = {}
  for fname, spec in config.specs.items():
    table = tables[spec.table_name or fname].to(torch.float32).cpu()
    vals, offs, w = inputs.feature(fname)
    vals, offs = vals.cpu().long(), offs.cpu()
    w = torch.ones(vals.numel()) if w is None else w.cpu().to(torch.float32)
    B = offs.numel() - 1
    lens = (offs[1:] - offs[:-1])
    bag = torch.repeat_interleave(torch.arange(B), lens)
    rows = table[vals] * w[:, None]
    if spec.max_sequence_length is not None:
      L = spec.max_sequence_length
      seq = torch.zeros(B, L, table.shape[1])
      pos = torch.arange(vals.numel()) - offs[:-1][bag]
      keep = pos < L
      seq[bag[keep], pos[keep]] = rows[keep]
      out[fname] = seq
      continue
    pooled = torch.zeros(B, table.shape[1]).index_add_(0, bag, rows)
    if spec.combiner == "mean":
      den = torch.zeros(B).index_add_(0, bag, w)
      pooled = torch.where(den[:, None] != 0, pooled / den[:, None].clamp_min(1e-30), torch.zeros(()))
    elif spec.combiner == "sqrtn":
      den = torch.sqrt(torch.zeros(B).index_add_(0, bag, w * w))
      pooled = torch.where(den[:, None] != 0, pooled / den[:, None].clamp_min(1e-30), torch.zeros(()))
    out[fname] = pooled
  return out
