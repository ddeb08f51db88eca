"""Multi-process (gloo, world_size 2 and 3) tests of the sharded-embedding plumbing, gradient
averaging and the tiny DLRM-DCNv2 job.  The reference has no multi-process test at all."""
import os

import pytest
import torch

from tests import dist_utils


def _single(placements, opt, steps=3):
  from tests import dist_workers
  return dist_workers.sharded_embedding_steps(0, 1, "cpu", "collective", placements, opt, steps)


@pytest.mark.parametrize("placements,opt", [
    (["row_wise", "row_wise", "row_wise", "row_wise"], "rowwise_adagrad"),
    (["table_wise", "row_wise", "table_wise", "column_wise"], "adam"),
    (["column_wise", "table_wise", "row_wise", "table_wise"], "sgd")])
@pytest.mark.parametrize("world", [2])
def test_sharded_embedding_matches_single_process(world, placements, opt):
  ref = _single(placements, opt)
  res = dist_utils.run_ranks("sharded_embedding_steps", world, "gloo", "cpu", "collective", placements, opt, 3)
  per = 64 // world
  for step in range(3):
    got = torch.cat([r["outs"][step] for r in res], dim=0)
    torch.testing.assert_close(got, ref["outs"][step], atol=1e-5, rtol=1e-5)
  for name, t in ref["tables"].items():
    torch.testing.assert_close(res[0]["tables"][name], t, atol=2e-4, rtol=1e-4)
    torch.testing.assert_close(res[1]["tables"][name], t, atol=2e-4, rtol=1e-4)


def test_gradient_averaging_gloo():
  res = dist_utils.run_ranks("allreduce_grads", 2, "gloo", "cpu", [(33, 7), (5,), (1000,)])
  assert all(e < 1e-6 for r in res for e in r["max_rel_err"])


def test_tiny_dlrm_two_ranks_matches_loss_trend():
  res = dist_utils.run_ranks("dlrm_tiny_training", 2, "gloo", "cpu", 60)
  assert res[0]["ckpts"] == ["49", "59"]
  assert res[0]["loss"] < 0.62 and abs(res[0]["loss"] - res[1]["loss"]) < 0.1


def test_vocab_rank_sharded_gloo():
  res = dist_utils.run_ranks("vocab_rank_sharded", 2, "gloo", "cpu", 24, 32, 501)
  assert all(r["max_excess"] <= 0 for r in res), res


def test_sasrec_tiny_two_ranks():
  res = dist_utils.run_ranks("sequence_experiment", 2, "gloo", "cpu", "sasrec", 30)
  assert res[0]["train"]["loss"] < 1.45 and 0.0 <= res[0]["val"]["ndcg@10"] <= 1.0


def test_row_wise_table_saved_by_two_ranks_restores_on_one(tmp_path):
  """MOD-sharded tables and their optimizer slots written by a 2-rank job are restored by a 1-rank job."""
  from recml_b200 import ckpt, embedding as emb
  d = str(tmp_path / "ck")
  res = dist_utils.run_ranks("save_row_wise_tables", 2, "gloo", "cpu", d, -1)
  specs = {"a": emb.EmbeddingSpec(37, 8, combiner="sum"), "b": emb.EmbeddingSpec(10, 8, combiner="sum")}
  cfg = emb.ShardedEmbeddingConfig(specs, emb.AdagradOptimizerSpec(learning_rate=0.1), sharding_strategy="MOD",
                                   backend="collective")
  m = emb.ShardedEmbedding(cfg, device="cpu")
  got = ckpt.CheckpointManager(d, async_save=False).restore(1, target={"sharded": m.sharded_state_dict()})
  m.load_sharded_state_dict(got["sharded"])
  for n in specs:
    torch.testing.assert_close(m.gather_table(n), res[0]["tables"][n])
    torch.testing.assert_close(m.gather_table(n, "accumulator"), res[0]["slots"][n])


def test_ocdbt_checkpoint_of_two_ranks_restores_on_one(tmp_path):
  """The OCDBT form with one store per writing process (`ocdbt.process_0`, `ocdbt.process_1`): a stacked,
  MOD-sharded table written by 2 ranks is re-sharded into a 1-rank job."""
  import os
  from recml_b200 import ckpt, embedding as emb
  d = str(tmp_path / "ck")
  res = dist_utils.run_ranks("save_row_wise_tables", 2, "gloo", "cpu", d, -1, True)
  item = os.path.join(d, "1", "state")
  assert {"manifest.ocdbt", "ocdbt.process_0", "ocdbt.process_1"} <= set(os.listdir(item))
  specs = {"a": emb.EmbeddingSpec(37, 8, combiner="sum"), "b": emb.EmbeddingSpec(10, 8, combiner="sum")}
  cfg = emb.ShardedEmbeddingConfig(specs, emb.AdagradOptimizerSpec(learning_rate=0.1), sharding_strategy="MOD",
                                   backend="collective")
  m = emb.ShardedEmbedding(cfg, device="cpu")
  got = ckpt.CheckpointManager(d, async_save=False).restore(1, target={"sharded": m.sharded_state_dict()})
  m.load_sharded_state_dict(got["sharded"])
  for n in specs:
    torch.testing.assert_close(m.gather_table(n), res[0]["tables"][n])
    torch.testing.assert_close(m.gather_table(n, "accumulator"), res[0]["slots"][n])


def test_failed_shard_write_commits_nothing_on_any_rank(tmp_path):
  d = str(tmp_path / "ck")
  res = dist_utils.run_ranks("save_row_wise_tables", 2, "gloo", "cpu", d, 1)
  assert res[0]["raised"] == "RuntimeError" and res[1]["raised"] == "OSError"
  for r in res:
    assert r["steps"] == [1]                           # the good checkpoint survives, step 2 does not exist
    assert not any(".orbax-checkpoint-tmp-" in n for n in r["listing"])


def _replicated_reference(steps, with_tp=False):
  from tests import dist_workers
  return dist_workers.sharded_state_training(0, 1, "cpu", [], 1, None, steps, None, with_tp)


RULES = [(r"b\.weight", ("model", None)), (r"b\.bias", ("model",)), (r"c\.weight", (None, "model"))]


def test_sharded_state_matches_replicated_run_two_ranks(tmp_path):
  """mesh (data 1) x (model 2): parameters sharded over "model" are gathered before use, their gradients cut
  back onto the shards, Adam slots are shard-sized, global-norm clipping sees the whole gradient, and the
  checkpoint stores the full arrays."""
  ref = _replicated_reference(4)
  res = dist_utils.run_ranks("sharded_state_training", 2, "gloo", "cpu", [("data", 1), ("model", 2)], 1, RULES, 4,
                             str(tmp_path / "ck"), False)
  for r in res:
    assert r["shapes"]["b.weight"] == (8, 16) and r["shapes"]["b.bias"] == (8,) and r["shapes"]["c.weight"] == (1, 8)
    assert r["slot_shapes"]["b.weight"] == (8, 16)
    assert r["restored_ok"]
    torch.testing.assert_close(torch.tensor(r["losses"]), torch.tensor(ref["losses"]), rtol=1e-5, atol=1e-6)
    for k, v in ref["full"].items():
      torch.testing.assert_close(r["full"][k], v, rtol=1e-4, atol=1e-6)
  assert res[0]["stored"]["b.weight"] == (16, 16) and res[0]["stored"]["c.weight"] == (1, 16)


def test_data_by_model_mesh_on_four_ranks():
  """mesh (data 2) x (model 2): the batch is split over "data", parameters over "model"."""
  ref = _replicated_reference(3)
  res = dist_utils.run_ranks("sharded_state_training", 4, "gloo", "cpu", [("data", 2), ("model", 2)], 1, RULES, 3, "",
                             False)
  for r in res:
    for k, v in ref["full"].items():
      torch.testing.assert_close(r["full"][k], v, rtol=1e-4, atol=1e-5)


def test_fully_sharded_data_parallel_two_ranks():
  """One data axis that also shards the parameters: gradients of different batches are reduce-scattered."""
  ref = _replicated_reference(3)
  rules = [(r"b\.weight", ("data", None)), (r"a\.weight", (None, "data"))]
  res = dist_utils.run_ranks("sharded_state_training", 2, "gloo", "cpu", [("data", 2)], 1, rules, 3, "", False)
  for r in res:
    assert r["shapes"]["b.weight"] == (8, 16) and r["shapes"]["a.weight"] == (16, 4)
    for k, v in ref["full"].items():
      torch.testing.assert_close(r["full"][k], v, rtol=1e-4, atol=1e-5)


def test_tensor_parallel_mlp_matches_dense_two_ranks():
  """Column-parallel + row-parallel layers on 2 ranks follow the single-process run of the same layers."""
  ref = _replicated_reference(3, with_tp=True)
  res = dist_utils.run_ranks("sharded_state_training", 2, "gloo", "cpu", [("data", 1), ("model", 2)], 1, [], 3, "", True)
  for r in res:
    torch.testing.assert_close(torch.tensor(r["losses"]), torch.tensor(ref["losses"]), rtol=1e-5, atol=1e-6)
    for k, v in ref["full"].items():
      torch.testing.assert_close(r["full"][k], v, rtol=1e-4, atol=1e-6)


def test_q_sequence_sharded_attention_matches_unsharded():
  """The op's sequence-sharded mode on 2 gloo ranks (causal, inclusive window, segment ids) equals the
  single-process op in outputs and in the gradients of q, k and v."""
  from recml_b200.ops import hstu_attention as A
  g = torch.Generator().manual_seed(3)
  B, L, H, Dh = 2, 24, 2, 8
  q, k, v = (torch.randn(B, L, H, Dh, generator=g).requires_grad_() for _ in range(3))
  seg = torch.tensor([[0] * 10 + [1] * 14, [0] * 24])
  go = torch.randn(B, L, H, Dh, generator=g)
  ref = A.pointwise_attention("causal", q, k, v, q_segment_ids=seg, sliding_window_size=6, scale=0.3)
  ref.backward(go)
  res = dist_utils.run_ranks("q_sharded_attention", 2, "gloo", "cpu")
  torch.testing.assert_close(torch.cat([r["out"] for r in res], dim=1), ref.detach())
  for i, t in enumerate((q, k, v)):
    torch.testing.assert_close(torch.cat([r["grads"][i] for r in res], dim=1), t.grad, rtol=1e-4, atol=1e-6)


def test_sliding_window_is_inclusive_like_the_reference_local_mask():
  from recml_b200.ops import hstu_attention as A
  m = A.attention_mask("causal", 8, 8, sliding_window_size=2)
  assert m[5].tolist() == [False, False, False, True, True, True, False, False]      # keys 3, 4, 5: w + 1 of them
  f = A.attention_mask("full", 8, 8, sliding_window_size=1)
  assert f[4].tolist() == [False, False, False, True, True, True, False, False]


def test_asynchronous_save_from_two_ranks(tmp_path):
  """`save` returns before the slower rank has written its shard, the checkpoint holds the values of the moment of
  the call although they changed meanwhile, and the staging directory's marker files are gone after the commit."""
  res = dist_utils.run_ranks("async_multi_rank_save", 2, "gloo", "cpu", str(tmp_path / "ck"), -1)
  for r, out in enumerate(res):
    assert out["raised"] is None and out["steps"] == [1] and out["listing"] == ["1"], out
    assert out["returned_after"] < 0.6, out["returned_after"]        # the slower writer alone takes 1 s
    torch.testing.assert_close(out["shard"], torch.full((4, 3), float(r + 1)))
    torch.testing.assert_close(out["whole"], torch.arange(6, dtype=torch.float32))
  assert not [n for n in os.listdir(tmp_path / "ck" / "1") if n.startswith(".rank_")]


def test_asynchronous_save_commits_nothing_when_a_rank_fails(tmp_path):
  res = dist_utils.run_ranks("async_multi_rank_save", 2, "gloo", "cpu", str(tmp_path / "ck"), 1)
  assert "disk full" in res[1]["raised"] and "nothing was committed" in res[0]["raised"]
  for out in res:
    assert out["steps"] == [] and out["listing"] == []
