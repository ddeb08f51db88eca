"""2-GPU tests of the fused compute+collective kernels against single-process CPU references.
Run on a box with two or more B200s; every peer wait in the kernels is bounded."""
import pytest
import torch

from tests import dist_utils

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _single(placements, opt, steps=3):
  from tests import dist_workers
  return dist_workers.sharded_embedding_steps(0, 1, "cpu", "collective", placements, opt, steps)


@pytest.mark.parametrize("placements,opt", [
    (["row_wise", "row_wise", "row_wise", "row_wise"], "rowwise_adagrad"),
    (["table_wise", "row_wise", "table_wise", "column_wise"], "adam"),
    (["table_wise", "table_wise", "table_wise", "table_wise"], "sgd")])
def test_fused_embedding_two_gpus(placements, opt):
  ref = _single(placements, opt)
  res = dist_utils.run_ranks("sharded_embedding_steps", 2, "nccl", "cuda", "fused", placements, opt, 3)
  for step in range(3):
    got = torch.cat([r["outs"][step] for r in res], dim=0)
    torch.testing.assert_close(got, ref["outs"][step], atol=3e-2, rtol=3e-2)
  for name, t in ref["tables"].items():
    torch.testing.assert_close(res[0]["tables"][name], t, atol=5e-3, rtol=5e-3)


@pytest.mark.parametrize("nvls", [False, True])
def test_fused_allreduce_two_gpus(nvls):
  """Peer-load two-shot reduce and the in-switch `multimem` reduce (taken only when the symmetric
  buffer has a multicast mapping) against NCCL's all-reduce."""
  res = dist_utils.run_ranks("allreduce_grads", 2, "nccl", "cuda", [(333, 77), (5,), (100000,), (1, 9), (2048, 2048)], nvls)
  assert res[0]["reducer"] == "FusedNvlinkReducer"
  assert all(e < 1e-2 for r in res for e in r["max_rel_err"]), res   # bf16 wire format
  print("fused all-reduce", {k: res[0][k] for k in ("nvls", "multicast", "ms")})


def test_dlrm_tiny_two_gpus():
  res = dist_utils.run_ranks("dlrm_tiny_training", 2, "nccl", "cuda", 60)
  assert res[0]["loss"] < 0.62


def test_dlrm_tiny_two_gpus_cuda_graph():
  res = dist_utils.run_ranks("dlrm_tiny_training", 2, "nccl", "cuda", 60, True)
  assert res[0]["loss"] < 0.62


def test_vocab_rank_two_gpus():
  res = dist_utils.run_ranks("vocab_rank_sharded", 2, "nccl", "cuda", 256, 256, 30011)
  assert all(r["max_excess"] <= 0 and r["exact"] > 0.9 for r in res), res


@pytest.mark.parametrize("which", ["sasrec", "hstu"])
def test_sequence_experiments_two_gpus(which):
  res = dist_utils.run_ranks("sequence_experiment", 2, "nccl", "cuda", which, 30)
  assert res[0]["train"]["loss"] == res[0]["train"]["loss"]   # finite


def test_sharded_state_partitioner_two_gpus(tmp_path):
  """mesh (data 1) x (model 2) over NCCL: a model whose layers are sharded over "model" (gathered before use,
  gradients cut back onto the shards, shard-sized Adam slots, global-norm clipping across shards) follows the
  replicated single-process run, and its checkpoint restores."""
  from tests import dist_workers
  rules = [(r"b\.weight", ("model", None)), (r"b\.bias", ("model",)), (r"c\.weight", (None, "model"))]
  # The replicated run uses the same GPU kernels.  bf16 products and atomically accumulated weight gradients are
  # not bit-reproducible between two runs, and Adam turns a sign flip of a tiny gradient into a full learning-rate
  # step, so after four steps the runs agree to a few learning rates (the tight comparison is the gloo test's).
  ref = dist_workers.sharded_state_training(0, 1, "cuda", [], 1, None, 4, None, False)
  res = dist_utils.run_ranks("sharded_state_training", 2, "nccl", "cuda", [("data", 1), ("model", 2)], 1, rules, 4,
                             str(tmp_path / "ck"), False)
  for r in res:
    assert r["shapes"]["b.weight"] == (8, 16) and r["slot_shapes"]["b.weight"] == (8, 16) and r["restored_ok"]
    torch.testing.assert_close(torch.tensor(r["losses"]), torch.tensor(ref["losses"]), rtol=5e-2, atol=5e-3)
    for k, v in ref["full"].items():
      torch.testing.assert_close(r["full"][k], v, rtol=0, atol=5e-2)
