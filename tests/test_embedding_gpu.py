"""Fused sharded-embedding kernels (1 GPU) vs the torch/collective backend on CPU."""
import numpy as np
import pytest
import torch

from recml_b200 import embedding as emb
from recml_b200.data import synthetic
from recml_b200.ops import _lib

pytestmark = pytest.mark.gpu

OPTS = [emb.RowWiseAdagradOptimizerSpec(0.05), emb.SGDOptimizerSpec(0.1), emb.AdagradOptimizerSpec(0.05),
        emb.AdamOptimizerSpec(0.01), emb.RowWiseAdamOptimizerSpec(0.01), emb.LaPropOptimizerSpec(0.01),
        emb.FTRLOptimizerSpec(0.05), emb.AdagradMomentumOptimizerSpec(0.05)]


def _pair(specs, opt):
  cfg_g = emb.ShardedEmbeddingConfig(specs, opt, backend="fused", seed=3)
  cfg_c = emb.ShardedEmbeddingConfig(specs, opt, backend="collective", seed=3)
  g = emb.ShardedEmbedding(cfg_g, device="cuda")
  c = emb.ShardedEmbedding(cfg_c, device="cpu")
  for name in g.plan.tables:
    c.load_table(name, g.gather_table(name).cpu())
  return g, c


def _batch(rng, B, vocabs, bags, weights=False, ragged=False):
  feats, ws = {}, {}
  for i, (v, b) in enumerate(zip(vocabs, bags)):
    rows = []
    for _ in range(B):
      n = int(rng.integers(0, b + 1)) if ragged else b
      rows.append(synthetic.zipf_ids(rng, v, (n,), 1.05).tolist())
    feats[f"f{i}"] = rows
    ws[f"f{i}"] = [[float(x) for x in rng.random(len(r)) + 0.5] for r in rows]
  return emb.KeyedJagged.from_lists(feats, ws if weights else None)


@pytest.mark.parametrize("opt", OPTS, ids=lambda o: o.kind)
def test_forward_backward_matches_reference(opt):
  rng = np.random.default_rng(0)
  vocabs, bags, D, B = [50, 1000, 7], [3, 40, 1], 128, 192
  specs = {f"f{i}": emb.EmbeddingSpec(v, D, combiner="sum") for i, v in enumerate(vocabs)}
  g, c = _pair(specs, opt)
  for step in range(3):
    kjt = _batch(rng, B, vocabs, bags)
    og = g(kjt.to_device(torch.device("cuda")))
    oc = c(kjt)
    torch.testing.assert_close(og.float().cpu(), oc, atol=2e-2, rtol=2e-2)
    grad = torch.randn(oc.shape) * 0.1
    grad = grad.to(torch.bfloat16).float()
    oc.backward(grad)
    og.backward(grad.cuda().to(og.dtype))
    torch.cuda.synchronize()
    _lib.check_status()
    for name in g.plan.tables:
      torch.testing.assert_close(g.gather_table(name).cpu(), c.gather_table(name), atol=3e-3, rtol=3e-3)


@pytest.mark.parametrize("D", [16, 64, 256])
@pytest.mark.parametrize("combiner", ["mean", "sqrtn"])
def test_combiners_weights_ragged(D, combiner):
  rng = np.random.default_rng(1)
  vocabs, bags, B = [33, 400], [5, 17], 96
  specs = {f"f{i}": emb.EmbeddingSpec(v, D, combiner=combiner) for i, v in enumerate(vocabs)}
  g, c = _pair(specs, emb.RowWiseAdagradOptimizerSpec(0.05))
  kjt = _batch(rng, B, vocabs, bags, weights=True, ragged=True)
  og, oc = g(kjt.to_device(torch.device("cuda"))), c(kjt)
  torch.testing.assert_close(og.float().cpu(), oc, atol=2e-2, rtol=2e-2)
  grad = (torch.randn(oc.shape) * 0.1).to(torch.bfloat16).float()
  oc.backward(grad)
  og.backward(grad.cuda().to(og.dtype))
  torch.cuda.synchronize()
  _lib.check_status()
  for name in g.plan.tables:
    torch.testing.assert_close(g.gather_table(name).cpu(), c.gather_table(name), atol=3e-3, rtol=3e-3)


def test_hot_rows_cross_chunk_reduction():
  """A 3-row table hit by 20k ids: every run of equal rows spans hundreds of 32-entry chunks."""
  rng = np.random.default_rng(2)
  specs = {"f0": emb.EmbeddingSpec(3, 128, combiner="sum"), "f1": emb.EmbeddingSpec(100000, 128, combiner="sum")}
  g, c = _pair(specs, emb.RowWiseAdagradOptimizerSpec(0.05))
  B = 2048
  kjt = emb.KeyedJagged.from_dense({"f0": rng.integers(0, 3, (B, 10)), "f1": synthetic.zipf_ids(rng, 100000, (B, 4))})
  og, oc = g(kjt.to_device(torch.device("cuda"))), c(kjt)
  grad = (torch.randn(oc.shape) * 0.05).to(torch.bfloat16).float()
  oc.backward(grad)
  og.backward(grad.cuda().to(og.dtype))
  torch.cuda.synchronize()
  _lib.check_status()
  for name in g.plan.tables:
    torch.testing.assert_close(g.gather_table(name).cpu(), c.gather_table(name), atol=5e-3, rtol=5e-3)
  # scratch lines must be back to zero for the next step
  assert float(g._backend.stacks[0]["scratch"].abs().max()) == 0.0


def test_sequence_feature_no_pooling():
  rng = np.random.default_rng(3)
  specs = {"s": emb.EmbeddingSpec(500, 64, max_sequence_length=6), "p": emb.EmbeddingSpec(50, 64, combiner="sum")}
  g, c = _pair(specs, emb.SGDOptimizerSpec(0.1))
  kjt = emb.KeyedJagged.from_lists({"s": [list(rng.integers(0, 500, int(rng.integers(0, 9)))) for _ in range(40)],
                                    "p": [list(rng.integers(0, 50, 3)) for _ in range(40)]})
  og, oc = g(kjt.to_device(torch.device("cuda"))), c(kjt)
  for k in oc:
    torch.testing.assert_close(og[k].float().cpu(), oc[k], atol=2e-2, rtol=2e-2)


def test_out_of_range_ids_are_reported_not_dereferenced():
  """An id beyond the vocabulary must neither be read nor update anything: the kernel records it and the
  host raises at the next status check."""
  import numpy as np
  import torch
  from recml_b200 import embedding as emb
  from recml_b200.ops import _lib
  spec = {"f": emb.EmbeddingSpec(100, 64, combiner="sum")}
  m = emb.ShardedEmbedding(emb.ShardedEmbeddingConfig(spec, emb.SGDOptimizerSpec(0.1)), device="cuda")
  _lib.check_status(torch.device("cuda"))
  values = torch.tensor([3, 5, 100_000, 7], dtype=torch.int32)
  offsets = torch.tensor([0, 2, 4], dtype=torch.int32)
  kjt = emb.KeyedJagged(("f",), values, offsets, None, 2).to_device(torch.device("cuda"))
  out = m(kjt)
  table = m.gather_table("f")
  ref1 = table[5] + table[3]
  ref2 = table[7]                         # the bad id contributes nothing
  torch.testing.assert_close(out.reshape(2, 64).float()[0], ref1.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2)
  torch.testing.assert_close(out.reshape(2, 64).float()[1], ref2.to(torch.bfloat16).float(), rtol=2e-2, atol=2e-2)
  with pytest.raises(_lib.DeviceStatusError, match="outside its table"):
    _lib.check_status(torch.device("cuda"))
  _lib.check_status(torch.device("cuda"))  # the status word was cleared


def test_id_dropping_counts_overflow_instead_of_failing():
  """The occurrence lists are sized from the first batch.  A later batch with far more ids overflows them: with
  `allow_id_dropping` the surplus ids are left out of the lookup and counted (reference
  `recml/layers/linen/sparsecore.py:107-108`), without it the overflow is an error at the next status check."""
  dev = torch.device("cuda")
  spec = {"f": emb.EmbeddingSpec(5000, 64, combiner="sum")}
  rng = np.random.default_rng(5)
  small = emb.KeyedJagged.from_lists({"f": [list(rng.integers(0, 5000, 2)) for _ in range(256)]})
  big = emb.KeyedJagged.from_lists({"f": [list(rng.integers(0, 5000, 40)) for _ in range(256)]})
  for allow in (True, False):
    m = emb.ShardedEmbedding(emb.ShardedEmbeddingConfig(spec, emb.SGDOptimizerSpec(0.1), allow_id_dropping=allow),
                             device="cuda")
    m(small.to_device(dev)).sum().backward()
    torch.cuda.synchronize()
    _lib.check_status(dev)
    before = m.gather_table("f").clone()
    out = m(big.to_device(dev))
    out.float().sum().backward()
    torch.cuda.synchronize()
    if allow:
      _lib.check_status(dev)
      cap = m._backend.stacks[0]["occ_cap"]
      assert m._backend.dropped_ids() == 256 * 40 - cap
      assert bool(torch.isfinite(out.float()).all())
      assert float((m.gather_table("f") - before).abs().max()) > 0       # the ids that fitted were trained
    else:
      with pytest.raises(_lib.DeviceStatusError):
        _lib.check_status(dev)
      _lib.check_status(dev)
