"""Sharding planner: decides where every embedding table lives.

The reference has one strategy — MOD row sharding of stacked tables over all
SparseCores, row i on shard (i % S + rotation) % S at local row i // S — plus a manual
vocabulary threshold below which a table is a replicated dense layer
(`recml/inference/models/jax/DLRM_DCNv2/dlrm_main.py:129-131`).  On an NVSwitch box all
peers are equidistant, so placement only has to balance (a) HBM bytes and (b) gather
work per rank:

  ROW_WISE     rows MOD-sharded over all ranks (large tables; spreads hot rows)
  TABLE_WISE   whole table on one rank (medium tables; one pooled vector per bag moves)
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
                row_wise_min_bytes: int = 256 << 20, replicate_max_rows: int = 0,
                column_wise: Sequence[str] = (), overrides: Mapping[str, Placement] | None = None,
                default: Placement | None = None) -> ShardingPlan:
  """Greedy plan.  Large tables are row-sharded; the rest go table-wise to the rank with
  the least accumulated gather cost (ids per sample × dim), largest first."""
  overrides = dict(overrides or {})
  ids_per_sample = ids_per_sample or {}
  plans: dict[str, TablePlan] = {}
  load = [0.0] * world
  rot = 0
  rw_cost = 0.0
  order = sorted(tables, key=lambda t: -(ids_per_sample.get(t.name, 1.0) * t.embedding_dim))
  for t in order:
    size = t.vocabulary_size * t.embedding_dim * 4
    p = overrides.get(t.name)
    if p is None:
      if world == 1:
        p = Placement.TABLE_WISE
      elif t.name in column_wise:
        p = Placement.COLUMN_WISE
      elif default is not None:
        p = default
      elif t.vocabulary_size <= replicate_max_rows:
        p = Placement.REPLICATED
      elif size >= row_wise_min_bytes:
        p = Placement.ROW_WISE
      else:
        p = Placement.TABLE_WISE
    cost = ids_per_sample.get(t.name, 1.0) * t.embedding_dim
    tp = TablePlan(t.name, t.vocabulary_size, t.embedding_dim, p)
    if p is Placement.ROW_WISE:
      tp.rotation = rot % world
      rot += 1
      tp.local_rows = _local_rows(t.vocabulary_size, world, rank, tp.rotation)
      tp.local_dim = t.embedding_dim
      rw_cost += cost / world
    elif p is Placement.TABLE_WISE:
      tp.owner = min(range(world), key=lambda r: load[r])
      load[tp.owner] += cost
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
