"""Sharding planner: decides where every embedding table lives.

The reference has one strategy — MOD row sharding of stacked tables over all
SparseCores, row i on shard (i % S + rotation) % S at local row i // S — plus a manual
vocabulary threshold below which a table is a replicated dense layer
(`recml/inference/models/jax/DLRM_DCNv2/dlrm_main.py:129-131`).  On an NVSwitch box all
peers are equidistant and one GPU holds 180 GB, so placement is driven by traffic and
gather balance, not by fitting a table:

  TABLE_WISE   whole table on one rank: ONE pooled vector per bag crosses NVLink in the
               forward and one gradient vector in the backward (the default)
  ROW_WISE     rows MOD-sharded over all ranks: every rank sends a partial per bag, W times
               the traffic, so only tables whose gather work would unbalance the ranks
               (cost above `hot_fraction` of the per-rank mean) or that exceed
               `table_wise_max_bytes` are split
  COLUMN_WISE  every rank holds a slice of the embedding dim (few-row, very hot tables)
  REPLICATED   every rank holds the table; its gradient joins the dense all-reduce

Tables with equal (local dim, optimizer) are STACKED into one buffer per rank so the
lookup and update kernels address one array with a per-table row offset.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Mapping, Sequence

from recml_b200.embedding import specs as specs_lib


class Placement(enum.Enum):
  ROW_WISE = "row_wise"
  TABLE_WISE = "table_wise"
  COLUMN_WISE = "column_wise"
  REPLICATED = "replicated"


@dataclasses.dataclass
class TablePlan:
  name: str
  vocab: int
  dim: int
  placement: Placement
  owner: int = 0           # TABLE_WISE: owning rank
  rotation: int = 0        # ROW_WISE: shard rotation
  stack: int = -1          # index of the stack holding this table's local rows
  row_base: int = 0        # first row of this table inside the stack (local)
  local_rows: int = 0      # rows stored on THIS rank
  local_dim: int = 0       # columns stored on this rank
  col_lo: int = 0

  def owner_of(self, ids, world: int):
    """Vectorised owner rank of each id (ROW_WISE)."""
    return (ids % world + self.rotation) % world


@dataclasses.dataclass
class StackPlan:
  dim: int
  optimizer: specs_lib.OptimizerSpec
  tables: list[str]
  rows: int = 0            # local rows on this rank


@dataclasses.dataclass
class ShardingPlan:
  world: int
  rank: int
  tables: dict[str, TablePlan]
  stacks: list[StackPlan]

  def bytes_on_rank(self, slot_bytes_per_row=lambda st: 4) -> int:
    return sum(st.rows * st.dim * 4 for st in self.stacks)


def _local_rows(vocab: int, world: int, rank: int, rotation: int) -> int:
  # row i lives on (i % W + rot) % W  ⇒ rank r holds residue (r - rot) mod W
  res = (rank - rotation) % world
  return (vocab - res + world - 1) // world if vocab > res else 0


def plan_tables(tables: Sequence[specs_lib.TableSpec], world: int, rank: int, *,
                ids_per_sample: Mapping[str, float] | None = None,
                row_wise_min_bytes: int | None = None, replicate_max_rows: int = 0,
                column_wise: Sequence[str] = (), overrides: Mapping[str, Placement] | None = None,
                default: Placement | None = None, hot_fraction: float = 0.75,
                table_wise_max_bytes: int = 48 << 30, rank_budget_bytes: int = 140 << 30,
                hot_row_share: Mapping[str, float | Sequence[float]] | None = None,
                residue_stats: Mapping[str, Sequence[Sequence[float]]] | None = None,
                unique_row_cost: float = 8.0, imbalance_tolerance: float = 0.15) -> ShardingPlan:
  """Greedy plan.  Cost of a table = ids per sample × dim (its gather work and its wire
  bytes).  Tables hotter than `hot_fraction` × (total cost / world), or larger than
  `table_wise_max_bytes`, are row-sharded; the rest go table-wise, largest cost first, to
  the rank with the least accumulated cost that still has `rank_budget_bytes` of room.
  `row_wise_min_bytes`, when given, replaces the cost rule with a plain size threshold.
  `hot_row_share[table]` is the share of a table's ids that hit its most frequent row, or a sequence with the
  shares of rows 0, 1, 2, ... (from recorded statistics or a known id distribution).  Row sharding spreads the
  rows evenly but not the ids: the rank that holds row k of a skewed table carries that row's share on top of
  its 1 / world of the rest, and the greedy pass gives it fewer whole tables in exchange.
  `residue_stats[table] = (ids[world], distinct[world])`, measured on a batch and expressed per sample, says how
  many ids and how many DISTINCT ids fall into each residue class `id % world`.  With it the cost of a table is
  ids + `unique_row_cost` x distinct ids (a distinct row costs a read-modify-write of the row and its optimizer
  state, and a cache miss in the lookup: about eight times an occurrence in the measured update kernel), a
  row-sharded table loads rank (q + rotation) % world with class q's cost, and its rotation is the one that
  keeps the most loaded rank lowest.  Tables without statistics use `ids_per_sample` / `hot_row_share`.
  Going through the tables from the costliest down, a table is also row-sharded when the rank that held it whole
  would, with its share of the tables row-sharded so far, exceed the mean load by more than
  `imbalance_tolerance`: no assignment of whole tables can hide such a table."""
  overrides = dict(overrides or {})
  ids_per_sample = ids_per_sample or {}
  plans: dict[str, TablePlan] = {}
  load = [0.0] * world
  used = [0] * world
  rot = 0
  residue_stats = dict(residue_stats or {})

  def class_costs(t):       # cost of each residue class of a table with statistics
    occ, uniq = residue_stats[t.name]
    return [(float(occ[q]) + unique_row_cost * float(uniq[q])) * t.embedding_dim for q in range(world)]

  def cost_of(t):
    if t.name in residue_stats and len(residue_stats[t.name][0]) == world:
      return sum(class_costs(t))
    return ids_per_sample.get(t.name, 1.0) * t.embedding_dim
  mean_cost = sum(cost_of(t) for t in tables) / max(world, 1)
  order = sorted(tables, key=lambda t: -cost_of(t))

  def row_bytes(t):
    return t.embedding_dim * 4 + t.optimizer.slot_bytes_per_row(t.embedding_dim)

  def auto(t):
    size = t.vocabulary_size * row_bytes(t)
    if world == 1:
      return Placement.TABLE_WISE
    if t.name in column_wise:
      return Placement.COLUMN_WISE
    if default is not None:
      return default
    if t.vocabulary_size <= replicate_max_rows:
      return Placement.REPLICATED
    if row_wise_min_bytes is not None:
      return Placement.ROW_WISE if size >= row_wise_min_bytes else Placement.TABLE_WISE
    if size > table_wise_max_bytes or (cost_of(t) > hot_fraction * mean_cost and t.vocabulary_size >= world):
      return Placement.ROW_WISE
    return Placement.TABLE_WISE

  chosen: dict[str, Placement] = {}
  total_cost = sum(cost_of(t) for t in tables)
  split_cost = 0.0          # cost of the tables row-sharded so far (every rank carries 1 / world of it)
  for t in order:
    p = overrides.get(t.name) or auto(t)
    if (p is Placement.TABLE_WISE and t.name not in overrides and world > 1 and default is None and
        row_wise_min_bytes is None and t.name not in column_wise and t.vocabulary_size >= world and
        cost_of(t) + split_cost / world > (1.0 + imbalance_tolerance) * total_cost / world):
      p = Placement.ROW_WISE
    if p is Placement.ROW_WISE:
      split_cost += cost_of(t)
    chosen[t.name] = p
  hot_row_share = dict(hot_row_share or {})
  # row-/column-wise tables load every rank equally (up to the hot row of a skewed row-wise table, which sits on
  # the rank its rotation names): account for them before the greedy pass.  Rotations are handed out in the
  # order of the second pass below.
  rot_preview = 0
  rot_of: dict[str, int] = {}
  for t in order:
    if chosen[t.name] is Placement.ROW_WISE and t.name in residue_stats and len(residue_stats[t.name][0]) == world:
      per = class_costs(t)
      best = min(range(world), key=lambda ro: (max(load[r] + per[(r - ro) % world] for r in range(world)), ro))
      for r in range(world):
        load[r] += per[(r - best) % world]
        used[r] += t.vocabulary_size * row_bytes(t) // world
      rot_of[t.name] = best
    elif chosen[t.name] is Placement.ROW_WISE:
      rot_of[t.name] = rot_preview % world
      shares = hot_row_share.get(t.name, ())
      shares = [float(shares)] if isinstance(shares, (int, float)) else [float(x) for x in shares]
      shares = [min(max(x, 0.0), 1.0) for x in shares]
      rest = max(1.0 - sum(shares), 0.0)
      for r in range(world):
        load[r] += cost_of(t) * rest / world
        used[r] += t.vocabulary_size * row_bytes(t) // world
      for k, x in enumerate(shares):          # row k lives on rank (k % world + rotation) % world
        load[(k % world + rot_preview) % world] += cost_of(t) * x
      rot_preview += 1
    elif chosen[t.name] is Placement.COLUMN_WISE:
      for r in range(world):
        load[r] += cost_of(t) / world
        used[r] += t.vocabulary_size * row_bytes(t) // world
  for t in order:
    p = chosen[t.name]
    size = t.vocabulary_size * row_bytes(t)
    if p is Placement.TABLE_WISE and world > 1 and t.name not in overrides:
      if not any(used[r] + size <= rank_budget_bytes for r in range(world)):
        p = Placement.ROW_WISE      # no rank has room for the whole table
        for r in range(world):
          load[r] += cost_of(t) / world
          used[r] += size // world
    cost = cost_of(t)
    tp = TablePlan(t.name, t.vocabulary_size, t.embedding_dim, p)
    if p is Placement.ROW_WISE:
      tp.rotation = rot_of.get(t.name, rot % world)
      if t.name not in residue_stats or len(residue_stats[t.name][0]) != world:
        rot += 1
      tp.local_rows = _local_rows(t.vocabulary_size, world, rank, tp.rotation)
      tp.local_dim = t.embedding_dim
    elif p is Placement.TABLE_WISE:
      fits = [r for r in range(world) if used[r] + size <= rank_budget_bytes] or list(range(world))
      tp.owner = min(fits, key=lambda r: load[r])
      load[tp.owner] += cost
      used[tp.owner] += size
      tp.local_rows = t.vocabulary_size if tp.owner == rank else 0
      tp.local_dim = t.embedding_dim
    elif p is Placement.COLUMN_WISE:
      if t.embedding_dim % world:
        raise ValueError(f"{t.name}: dim {t.embedding_dim} not divisible by world {world}")
      tp.local_dim = t.embedding_dim // world
      tp.col_lo = rank * tp.local_dim
      tp.local_rows = t.vocabulary_size
    else:
      tp.local_rows, tp.local_dim = t.vocabulary_size, t.embedding_dim
    plans[t.name] = tp
  # stacks: keep the caller's table order inside a stack for a stable layout
  stacks: list[StackPlan] = []
  by_name = {t.name: t for t in tables}
  for t in tables:
    tp = plans[t.name]
    if tp.placement is Placement.REPLICATED:
      continue
    for i, st in enumerate(stacks):
      if st.dim == tp.local_dim and st.optimizer == by_name[t.name].optimizer:
        tp.stack = i
        break
    else:
      stacks.append(StackPlan(tp.local_dim, by_name[t.name].optimizer, []))
      tp.stack = len(stacks) - 1
    st = stacks[tp.stack]
    tp.row_base = st.rows
    st.rows += tp.local_rows
    st.tables.append(t.name)
  return ShardingPlan(world, rank, plans, stacks)
