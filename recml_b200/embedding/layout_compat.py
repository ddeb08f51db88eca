"""Import / export of the reference's stacked, MOD-sharded table layout.

Checkpoints written by the reference store one array per table STACK of shape
`[num_shards * rows_per_shard, padded_dim]`, produced from the logical tables like this
(`jax_tpu_embedding/sparsecore/lib/nn/table_stacking.py:105-136, 350-373, 553-586`):

  1. pad the vocabulary to a multiple of `8 * num_shards` and the dim to a multiple of 8;
  2. MOD-shard: row i goes to shard `i % num_shards`, local row `i // num_shards`;
  3. rotate the shards of the k-th table of a stack by `k * rotation` (mod num_shards), so the hot
     low ids of different tables do not pile up on shard 0;
  4. stack: the table occupies local rows `[row_offset, row_offset + padded_vocab / num_shards)`
     of every shard, offsets accumulating in stacking order.
The stack is named by joining the table names with `_` (cut to 50 characters plus `...` and 12 hex
digits of its sha256 when longer, `table_stacking.py:727-759`).

`stack_layout` reproduces the settings, `to_reference_stack` / `from_reference_stack` convert
between logical tables and that array, so tables trained here can be exported to, and warm
started from, the reference's layout.  Everything is plain numpy on the host.
"""
from __future__ import annotations

import dataclasses
import hashlib
from typing import Mapping, Sequence

import numpy as np


def _round_up(x: int, m: int) -> int:
  return (x + m - 1) // m * m


@dataclasses.dataclass(frozen=True)
class TableInStack:
  name: str
  vocab: int
  dim: int
  padded_vocab: int
  padded_dim: int
  row_offset_in_shard: int
  shard_rotation: int


@dataclasses.dataclass(frozen=True)
class StackLayout:
  name: str
  num_shards: int
  padded_dim: int
  rows_per_shard: int
  tables: tuple[TableInStack, ...]

  def table(self, name: str) -> TableInStack:
    for t in self.tables:
      if t.name == name:
        return t
    raise KeyError(name)


def stack_name(table_names: Sequence[str], *, short: bool = True, max_len: int = 50, hash_len: int = 12) -> str:
  full = "_".join(table_names)
  if not short or len(full) <= max_len:
    return full
  return full[:max_len] + "..." + hashlib.sha256(full.encode("utf-8")).hexdigest()[:hash_len]


def stack_layout(tables: Sequence[tuple[str, int, int]], num_shards: int, *, rotation: int = 1,
                 name: str | None = None) -> StackLayout:
  """Settings of every `(name, vocab, dim)` table stacked in the given order.  `rotation` is the
  per-table shard rotation step (the reference uses the number of SparseCores per device)."""
  if not tables:
    raise ValueError("a stack needs at least one table")
  padded_dim = max(_round_up(d, 8) for _, _, d in tables)
  out, offset, rot = [], 0, 0
  for tname, vocab, dim in tables:
    pv = _round_up(vocab, 8 * num_shards)
    out.append(TableInStack(tname, vocab, dim, pv, padded_dim, offset, rot))
    offset += pv // num_shards
    rot = (rot + rotation) % num_shards
  return StackLayout(name or stack_name([t[0] for t in tables]), num_shards, padded_dim, offset, tuple(out))


def to_reference_stack(layout: StackLayout, tables: Mapping[str, np.ndarray], *, pad_value: float = 0.0) -> np.ndarray:
  """Logical tables → `[num_shards * rows_per_shard, padded_dim]` (shard-major)."""
  S = layout.num_shards
  stacked = np.full((S, layout.rows_per_shard, layout.padded_dim), pad_value, dtype=np.float32)
  for t in layout.tables:
    w = np.asarray(tables[t.name], dtype=np.float32)
    if w.shape != (t.vocab, t.dim):
      raise ValueError(f"table {t.name}: expected {(t.vocab, t.dim)}, got {w.shape}")
    padded = np.full((t.padded_vocab, t.padded_dim), pad_value, dtype=np.float32)
    padded[:t.vocab, :t.dim] = w
    per_shard = t.padded_vocab // S
    # [local row, shard, dim] → [shard, local row, dim]; shard s then moves to (s + rotation) % S
    sharded = padded.reshape(per_shard, S, t.padded_dim).transpose(1, 0, 2)
    rotated = np.roll(sharded, t.shard_rotation, axis=0)
    stacked[:, t.row_offset_in_shard:t.row_offset_in_shard + per_shard] = rotated
  return stacked.reshape(S * layout.rows_per_shard, layout.padded_dim)


def from_reference_stack(layout: StackLayout, stacked: np.ndarray) -> dict[str, np.ndarray]:
  """Inverse of `to_reference_stack`: un-stack, un-rotate, un-shard, un-pad."""
  S = layout.num_shards
  arr = np.asarray(stacked, dtype=np.float32)
  if arr.shape != (S * layout.rows_per_shard, layout.padded_dim):
    raise ValueError(f"stack {layout.name}: expected {(S * layout.rows_per_shard, layout.padded_dim)}, got {arr.shape}")
  arr = arr.reshape(S, layout.rows_per_shard, layout.padded_dim)
  out = {}
  for t in layout.tables:
    per_shard = t.padded_vocab // S
    piece = arr[:, t.row_offset_in_shard:t.row_offset_in_shard + per_shard]
    piece = np.roll(piece, -t.shard_rotation, axis=0)
    out[t.name] = piece.transpose(1, 0, 2).reshape(t.padded_vocab, t.padded_dim)[:t.vocab, :t.dim].copy()
  return out


def reference_location(layout: StackLayout, table: str, row: int) -> tuple[int, int]:
  """(shard, local row inside the stack) of a logical row: the addressing rule of
  `table_stacking.py:1216-1220`."""
  t = layout.table(table)
  return (row % layout.num_shards + t.shard_rotation) % layout.num_shards, row // layout.num_shards + t.row_offset_in_shard


def export_module(module, num_shards: int, *, rotation: int = 1, group_by_dim: bool = True
                  ) -> dict[str, tuple[StackLayout, np.ndarray]]:
  """All tables of a `ShardedEmbedding` in the reference layout: tables of equal padded dim share
  a stack (in the module's table order).  Collective when the module is sharded (it gathers)."""
  names = list(module.plan.tables)
  full = {n: module.gather_table(n).detach().cpu().numpy() for n in names}
  groups: dict[int, list[str]] = {}
  for n in names:
    key = _round_up(full[n].shape[1], 8) if group_by_dim else 0
    groups.setdefault(key, []).append(n)
  out = {}
  for members in groups.values():
    lay = stack_layout([(n, full[n].shape[0], full[n].shape[1]) for n in members], num_shards, rotation=rotation)
    out[lay.name] = (lay, to_reference_stack(lay, full))
  return out


def import_into_module(module, layout: StackLayout, stacked: np.ndarray) -> None:
  """Loads every table of a reference stack into a `ShardedEmbedding` (each rank keeps its part)."""
  import torch
  for name, w in from_reference_stack(layout, stacked).items():
    module.load_table(name, torch.from_numpy(w))
