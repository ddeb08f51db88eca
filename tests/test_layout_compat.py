"""Reference stacked-table layout (pad → MOD shard → rotate → stack) and the JSON spec side-car."""
import json

import numpy as np
import pytest
import torch

from recml_b200 import embedding as emb
from recml_b200.embedding import layout_compat as lc
from recml_b200.embedding import spec_sidecar


def test_stack_layout_settings_follow_reference_rules():
  lay = lc.stack_layout([("a", 10, 6), ("b", 100, 8), ("c", 33, 3)], num_shards=4, rotation=2)
  a, b, c = lay.tables
  assert (a.padded_vocab, b.padded_vocab, c.padded_vocab) == (32, 128, 64)      # multiples of 8*4
  assert lay.padded_dim == 8
  assert (a.row_offset_in_shard, b.row_offset_in_shard, c.row_offset_in_shard) == (0, 8, 40)
  assert (a.shard_rotation, b.shard_rotation, c.shard_rotation) == (0, 2, 0)   # (k*2) % 4
  assert lay.rows_per_shard == 56 and lay.name == "a_b_c"
  long = lc.stack_name([f"table_number_{i}" for i in range(8)])
  assert long.startswith("table_number_0_table_number_1_") and len(long) == 50 + 3 + 12


def test_round_trip_and_row_addressing():
  rng = np.random.default_rng(0)
  tabs = {"a": rng.normal(size=(10, 6)).astype(np.float32), "b": rng.normal(size=(100, 8)).astype(np.float32),
          "c": rng.normal(size=(33, 3)).astype(np.float32)}
  lay = lc.stack_layout([(n, *t.shape) for n, t in tabs.items()], num_shards=4, rotation=1)
  stacked = lc.to_reference_stack(lay, tabs)
  assert stacked.shape == (4 * lay.rows_per_shard, 8)
  back = lc.from_reference_stack(lay, stacked)
  for n in tabs:
    np.testing.assert_array_equal(back[n], tabs[n])
  # a logical row sits where the reference's addressing rule says
  per_shard = stacked.reshape(4, lay.rows_per_shard, 8)
  for name, row in (("a", 7), ("b", 42), ("b", 99), ("c", 0), ("c", 32)):
    shard, local = lc.reference_location(lay, name, row)
    np.testing.assert_array_equal(per_shard[shard, local, :tabs[name].shape[1]], tabs[name][row])
  with pytest.raises(ValueError):
    lc.from_reference_stack(lay, stacked[:-1])


def test_module_export_import_and_sidecar(tmp_path):
  specs = {"f0": emb.EmbeddingSpec(50, 16, combiner="sum"), "f1": emb.EmbeddingSpec(300, 16, combiner="mean"),
           "f2": emb.EmbeddingSpec(7, 8, combiner="sum")}
  cfg = emb.ShardedEmbeddingConfig(specs, emb.RowWiseAdagradOptimizerSpec(0.05), backend="collective")
  m = emb.ShardedEmbedding(cfg, device="cpu")
  exported = lc.export_module(m, num_shards=8)
  assert len(exported) == 2                      # one stack per padded dim
  m2 = emb.ShardedEmbedding(dataclasses_replace_seed(cfg, 7), device="cpu")
  assert not torch.equal(m2.gather_table("f1"), m.gather_table("f1"))
  for lay, arr in exported.values():
    lc.import_into_module(m2, lay, arr)
  for n in m.plan.tables:
    assert torch.equal(m2.gather_table(n), m.gather_table(n))
  path = spec_sidecar.write(m, str(tmp_path / "embedding_spec.json"), reference_shards=8)
  doc = spec_sidecar.read(path)
  assert {t["name"] for t in doc["tables"]} == {"f0", "f1", "f2"}
  assert [t.name for t in spec_sidecar.table_specs(doc)] == [t["name"] for t in doc["tables"]]
  opt = spec_sidecar.table_specs(doc)[0].optimizer
  assert opt.kind == "rowwise_adagrad" and opt.learning_rate == 0.05
  assert set(spec_sidecar.placement_overrides(doc).values()) == {emb.Placement.TABLE_WISE}
  lays = spec_sidecar.reference_layouts(doc)
  assert sorted(l.name for l in lays) == sorted(exported)
  with open(tmp_path / "bad.json", "w") as f:
    json.dump({"format": "other"}, f)
  with pytest.raises(ValueError):
    spec_sidecar.read(str(tmp_path / "bad.json"))


def dataclasses_replace_seed(cfg, seed):
  import dataclasses
  return dataclasses.replace(cfg, seed=seed)
