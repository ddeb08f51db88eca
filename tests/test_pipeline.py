"""Software pipelining of embedding and dense stages across steps."""
import numpy as np
import pytest
import torch
from torch import nn

from recml_b200 import embedding as emb
from recml_b200.training import pipeline


def _kjt(rng, B):
  lens = rng.integers(1, 4, B)
  off = np.zeros(B + 1, np.int32)
  off[1:] = np.cumsum(lens)
  return emb.KeyedJagged(("f",), torch.from_numpy(rng.integers(0, 40, off[-1]).astype(np.int32)), torch.from_numpy(off),
                         None, B)


def _make():
  cfg = emb.ShardedEmbeddingConfig({"f": emb.EmbeddingSpec(40, 8, combiner="sum")}, emb.SGDOptimizerSpec(0.5),
                                   backend="collective", seed=3)
  torch.manual_seed(0)
  return emb.ShardedEmbedding(cfg, device="cpu"), nn.Linear(8, 1)


def test_stage_order_and_results():
  log = []
  p = pipeline.PipelinedStep(lambda b: (log.append(("L", b)), f"a{b}")[1],
                             lambda a, b: (log.append(("D", b)), (f"g{b}", f"r{b}"))[1],
                             lambda g, a: log.append(("U", g, a)))
  outs = [p(i) for i in range(4)]
  outs.append(p.finalize())
  assert outs == [None, "r0", "r1", "r2", "r3"]
  assert log == [("L", 0), ("L", 1), ("D", 0), ("U", "g0", "a0"), ("L", 2), ("D", 1), ("U", "g1", "a1"), ("L", 3),
                 ("D", 2), ("U", "g2", "a2"), ("D", 3), ("U", "g3", "a3")]


def test_pipelined_training_matches_the_stale_schedule():
  rng = np.random.default_rng(0)
  batches = [{"ids": _kjt(rng, 6), "y": torch.randn(6, 1)} for _ in range(5)]

  def dense_fn_for(lin, opt):
    def dense_fn(acts, batch):
      opt.zero_grad()
      loss = ((lin(acts.reshape(6, 8).float()) - batch["y"]) ** 2).mean()
      loss.backward()
      opt.step()
      return loss, float(loss)
    return dense_fn

  e1, l1 = _make()
  p = pipeline.for_sharded_embedding(e1, dense_fn_for(l1, torch.optim.SGD(l1.parameters(), 0.1)), lambda b: b["ids"])
  losses = [p(b) for b in batches] + [p.finalize()]
  assert losses[0] is None and all(isinstance(x, float) for x in losses[1:])

  # the same schedule written out by hand: lookup(i) sees the updates of steps <= i-2
  e2, l2 = _make()
  dense2 = dense_fn_for(l2, torch.optim.SGD(l2.parameters(), 0.1))
  acts, ref = {}, []
  acts[0] = e2(batches[0]["ids"])
  for i in range(1, len(batches) + 2):
    if i - 2 >= 0 and (i - 2) in acts and hasattr(acts[i - 2], "_g"):
      acts[i - 2].backward(acts[i - 2]._g)
    if i < len(batches):
      acts[i] = e2(batches[i]["ids"])
    if i - 1 < len(batches):
      leaf = acts[i - 1].detach().requires_grad_(True)
      _, r = dense2(leaf, batches[i - 1])
      acts[i - 1]._g = leaf.grad
      ref.append(r)
  np.testing.assert_allclose(losses[1:], ref, rtol=1e-6)
  assert torch.allclose(e1.gather_table("f"), e2.gather_table("f"))
  assert torch.allclose(l1.weight, l2.weight)

  # and it differs from the unpipelined run (the staleness is real)
  e3, l3 = _make()
  dense3 = dense_fn_for(l3, torch.optim.SGD(l3.parameters(), 0.1))
  seq = []
  for b in batches:
    a = e3(b["ids"])
    leaf = a.detach().requires_grad_(True)
    _, r = dense3(leaf, b)
    a.backward(leaf.grad)
    seq.append(r)
  assert not np.allclose(seq, ref)


@pytest.mark.gpu
def test_pipelined_fused_backend_follows_the_collective_one():
  """The three-stage pipeline over the fused NVLink backend (two occurrence lists in flight, launch-time
  sequence numbers) gives the losses and tables of the same stale schedule run with the collective backend.
  (Plain SGD on the tables: a normalising optimizer turns the rounding of the bf16 activations into sign flips
  of near-zero row gradients, which says nothing about the schedule.)"""
  rng = np.random.default_rng(1)
  B, D = 256, 64
  def kjt():
    lens = rng.integers(1, 5, B)
    off = np.zeros(B + 1, np.int32)
    off[1:] = np.cumsum(lens)
    return emb.KeyedJagged(("f",), torch.from_numpy(rng.integers(0, 500, off[-1]).astype(np.int32)),
                           torch.from_numpy(off), None, B)
  batches = [{"ids": kjt(), "y": torch.randn(B, 1)} for _ in range(6)]

  def run(backend):
    cfg = emb.ShardedEmbeddingConfig({"f": emb.EmbeddingSpec(500, D, combiner="sum")},
                                     emb.SGDOptimizerSpec(0.5), backend=backend, seed=3)
    torch.manual_seed(0)
    e = emb.ShardedEmbedding(cfg, device="cuda")
    lin = nn.Linear(D, 1).cuda()
    opt = torch.optim.SGD(lin.parameters(), 0.05)

    def dense_fn(acts, batch):
      opt.zero_grad()
      loss = ((lin(acts.reshape(B, D).float()) - batch["y"].cuda()) ** 2).mean()
      loss.backward()
      opt.step()
      return loss, loss.detach()
    p = pipeline.for_sharded_embedding(e, dense_fn, lambda b: b["ids"].to_device(torch.device("cuda")),
                                       device=torch.device("cuda"))
    losses = [p(b) for b in batches] + [p.finalize()]
    torch.cuda.synchronize()
    return [float(x) for x in losses[1:]], e.gather_table("f").cpu()

  lf, tf_ = run("fused")
  lc, tc = run("collective")
  from recml_b200.ops import _lib
  _lib.check_status()
  np.testing.assert_allclose(lf, lc, rtol=2e-2, atol=2e-3)
  torch.testing.assert_close(tf_, tc, rtol=2e-2, atol=2e-3)
