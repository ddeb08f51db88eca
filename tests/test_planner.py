"""Embedding sharding planner: every table placed, hot / oversized tables split by rows, table-wise
tables balanced by cost under the memory budget, overrides and special placements honoured, and the
plan identical on every rank (each rank computes it on its own)."""
import numpy as np
import pytest

from recml_b200.embedding import planner as P, specs as S

CRITEO_VOCAB = [40_000_000, 39_060, 17_295, 7_424, 20_265, 3, 7_122, 1_543, 63, 40_000_000, 3_067_956, 405_282, 10,
                2_209, 11_938, 155, 4, 976, 14, 40_000_000, 40_000_000, 40_000_000, 590_152, 12_973, 108, 36]
CRITEO_HOT = [3, 2, 1, 2, 6, 1, 1, 1, 1, 7, 3, 8, 1, 6, 9, 5, 1, 1, 1, 12, 100, 27, 10, 3, 1, 1]


def _tables(vocab, dim=128):
  opt = S.RowWiseAdagradOptimizerSpec(learning_rate=0.01)
  return [S.TableSpec(f"t{i}", v, dim, opt) for i, v in enumerate(vocab)]


def test_criteo_geometry_on_eight_ranks():
  tables = _tables(CRITEO_VOCAB)
  ids = {f"t{i}": float(h) for i, h in enumerate(CRITEO_HOT)}
  plans = [P.plan_tables(tables, 8, r, ids_per_sample=ids) for r in range(8)]
  ref = plans[0]
  assert set(ref.tables) == {t.name for t in tables}
  for p in plans[1:]:                                   # the same decisions on every rank
    for name, tp in p.tables.items():
      assert (tp.placement, tp.owner, tp.rotation) == (ref.tables[name].placement, ref.tables[name].owner,
                                                        ref.tables[name].rotation)
  row_wise = {n for n, tp in ref.tables.items() if tp.placement is P.Placement.ROW_WISE}
  assert {"t20", "t21"} <= row_wise and len(row_wise) <= 6          # the bags of 100 and 27 ids dominate the cost
  # every row of every table is stored exactly once across the ranks
  for t in tables:
    rows = sum(p.tables[t.name].local_rows for p in plans)
    assert rows == t.vocabulary_size, (t.name, rows)
  # table-wise load: no rank carries more than twice the mean cost of the table-wise tables
  load = np.zeros(8)
  for n, tp in ref.tables.items():
    if tp.placement is P.Placement.TABLE_WISE:
      load[tp.owner] += ids[n] * 128
  assert load.max() <= 2.0 * load.mean() + 1e-9
  assert max(p.bytes_on_rank() for p in plans) < 140 << 30


def test_single_rank_keeps_everything_local():
  tables = _tables([1000, 50, 7])
  p = P.plan_tables(tables, 1, 0)
  assert all(tp.local_rows == t.vocabulary_size and tp.local_dim == t.embedding_dim
             for t, tp in ((t, p.tables[t.name]) for t in tables))


def test_overrides_replication_and_column_wise():
  tables = _tables([100_000, 64, 5_000, 900], dim=64)
  ids = {"t0": 10.0, "t1": 1.0, "t2": 0.5, "t3": 1.0}          # t2 is cold: well under the mean cost per rank
  p = [P.plan_tables(tables, 4, r, ids_per_sample=ids, overrides={"t0": P.Placement.ROW_WISE}, replicate_max_rows=100,
                     column_wise=["t3"]) for r in range(4)]
  assert p[0].tables["t0"].placement is P.Placement.ROW_WISE
  assert sum(x.tables["t0"].local_rows for x in p) == 100_000
  assert p[0].tables["t1"].placement is P.Placement.REPLICATED and all(x.tables["t1"].local_rows == 64 for x in p)
  assert p[0].tables["t3"].placement is P.Placement.COLUMN_WISE
  assert sum(x.tables["t3"].local_dim for x in p) == 64 and all(x.tables["t3"].local_rows == 900 for x in p)
  owners = {x.tables["t2"].owner for x in p}
  assert len(owners) == 1 and p[0].tables["t2"].placement is P.Placement.TABLE_WISE
  assert [x.tables["t2"].local_rows for x in p].count(5_000) == 1


def test_oversized_table_is_split_and_budget_is_respected():
  big = _tables([30_000_000, 30_000_000, 1000], dim=128)          # 15.4 GB each
  p = [P.plan_tables(big, 2, r, table_wise_max_bytes=8 << 30) for r in range(2)]
  assert all(p[0].tables[n].placement is P.Placement.ROW_WISE for n in ("t0", "t1"))
  q = [P.plan_tables(big, 2, r, rank_budget_bytes=20 << 30, hot_fraction=10.0) for r in range(2)]
  tw = [n for n in ("t0", "t1") if q[0].tables[n].placement is P.Placement.TABLE_WISE]
  assert len({q[0].tables[n].owner for n in tw}) == len(tw)       # two 15 GB tables cannot share a 20 GB rank


def test_hot_row_shares_offset_the_rank_that_holds_them():
  """Row sharding spreads rows, not ids: with the shares of the most frequent rows known, the greedy pass gives the
  ranks that hold them fewer whole tables, and the expected ids per rank even out (Criteo geometry, Zipf 1.05)."""
  import numpy as np
  from recml_b200.data import synthetic
  V, bags, W = synthetic.CRITEO_VOCAB_SIZES, synthetic.CRITEO_MULTI_HOT_SIZES, 8
  opt = S.RowWiseAdagradOptimizerSpec(learning_rate=0.01)
  tables = [S.TableSpec(name=f"t{i}", vocabulary_size=v, embedding_dim=128, optimizer=opt) for i, v in enumerate(V)]
  ids = {f"t{i}": float(b) for i, b in enumerate(bags)}

  def expected_ids(plan):
    load = np.zeros(W)
    for i, (v, b) in enumerate(zip(V, bags)):
      tp = plan.tables[f"t{i}"]
      if tp.placement is P.Placement.TABLE_WISE:
        load[tp.owner] += b
      else:
        ps = synthetic.zipf_head_shares(v, 1.05, 256)
        for k, pk in enumerate(ps):
          load[(k % W + tp.rotation) % W] += b * pk
        load += b * (1 - sum(ps)) / W
    return load

  even = P.plan_tables(tables, W, 0, ids_per_sample=ids)
  hot = {f"t{i}": synthetic.zipf_head_shares(v) for i, v in enumerate(V)}
  skewed = [P.plan_tables(tables, W, r, ids_per_sample=ids, hot_row_share=hot) for r in range(W)]
  a, b = expected_ids(even), expected_ids(skewed[0])
  assert a.max() / a.mean() > 1.12 and b.max() / b.mean() < 1.05
  for p in skewed[1:]:          # every rank derives the same plan
    assert {n: (t.placement, t.owner, t.rotation) for n, t in p.tables.items()} == \
        {n: (t.placement, t.owner, t.rotation) for n, t in skewed[0].tables.items()}


def test_residue_statistics_weigh_distinct_rows_and_split_what_cannot_be_hidden():
  """With per-class counts of ids and DISTINCT ids (what `embedding.stats.batch_residue_stats` measures), a table whose
  many distinct rows make it too costly for one rank is row-sharded although its id count alone is modest, and the
  ranks' costs (ids + 8 x distinct ids) even out."""
  from recml_b200.data import synthetic
  V, bags, W, B = synthetic.CRITEO_VOCAB_SIZES, synthetic.CRITEO_MULTI_HOT_SIZES, 8, 8192
  opt = S.RowWiseAdagradOptimizerSpec(learning_rate=0.01)
  tables = [S.TableSpec(name=f"t{i}", vocabulary_size=v, embedding_dim=128, optimizer=opt) for i, v in enumerate(V)]
  ids = {f"t{i}": float(b) for i, b in enumerate(bags)}
  rng = np.random.default_rng(0)
  draws = [synthetic.zipf_ids(rng, v, (B * b,), 1.05) for v, b in zip(V, bags)]
  stats = {f"t{i}": ((np.bincount(x % W, minlength=W) / B).tolist(),
                     (np.bincount(np.unique(x) % W, minlength=W) / B).tolist()) for i, x in enumerate(draws)}

  def cost(plan):
    c = np.zeros(W)
    for i, x in enumerate(draws):
      tp = plan.tables[f"t{i}"]
      owner = np.full(x.shape, tp.owner) if tp.placement is P.Placement.TABLE_WISE else (x % W + tp.rotation) % W
      for r in range(W):
        sel = x[owner == r]
        c[r] += sel.size + 8 * np.unique(sel).size
    return c

  plain = P.plan_tables(tables, W, 0, ids_per_sample=ids)
  informed = [P.plan_tables(tables, W, r, ids_per_sample=ids, residue_stats=stats) for r in range(W)]
  split = lambda plan: {n for n, t in plan.tables.items() if t.placement is P.Placement.ROW_WISE}
  assert split(plain) == {"t20", "t21"} and split(informed[0]) >= {"t20", "t21", "t19"} and len(split(informed[0])) <= 4
  a, b = cost(plain), cost(informed[0])
  assert b.max() / b.mean() < a.max() / a.mean() - 0.1
  for p in informed[1:]:
    assert {n: (t.placement, t.owner, t.rotation) for n, t in p.tables.items()} == \
        {n: (t.placement, t.owner, t.rotation) for n, t in informed[0].tables.items()}


def test_batch_residue_stats_counts_ids_and_distinct_ids_per_class():
  import torch
  from recml_b200 import embedding as emb
  kjt = emb.KeyedJagged.from_lists({"a": [[0, 4, 4], [1], [8, 9]], "b": [[3], [], [3, 7]]})
  st = emb.batch_residue_stats(kjt, 4)          # no process group: the local batch is the global one
  # feature a: ids 0 4 4 1 8 9 -> classes 0,0,0,1,0,1 ; distinct 0 4 1 8 9 -> classes 0,0,1,0,1
  assert st["a"][0] == [4 / 3, 2 / 3, 0.0, 0.0] and st["a"][1] == [3 / 3, 2 / 3, 0.0, 0.0]
  assert st["b"][0] == [0.0, 0.0, 0.0, 3 / 3] and st["b"][1] == [0.0, 0.0, 0.0, 2 / 3]
  assert emb.batch_residue_stats(kjt, 1) is None
