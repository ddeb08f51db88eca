"""DLRM experiment pieces that need no GPU."""
import numpy as np
import pytest


def test_feature_set_describes_the_model_geometry():
  """`FeatureSet` (`recml/examples/dlrm_experiment.py:44-98`): unique names, dense / sparse views, union; the
  Criteo feature set gives the benchmark geometry."""
  from recml_b200.data import synthetic
  from recml_b200.examples import dlrm_experiment as D
  fs = D.features()
  assert len(fs.dense_features()) == 13 and len(fs.sparse_features()) == 26
  cfg = D.ModelConfig.from_features(fs, num_cross_layers=2)
  assert cfg.vocab_sizes == tuple(synthetic.CRITEO_VOCAB_SIZES) and cfg.bag_sizes == tuple(synthetic.CRITEO_MULTI_HOT_SIZES)
  assert cfg.num_dense == 13 and cfg.embedding_dim == 128 and cfg.num_cross_layers == 2
  with pytest.raises(ValueError, match="unique"):
    D.FeatureSet([D.DenseFeature("a"), D.DenseFeature("a")])
  mixed = D.FeatureSet([D.SparseFeature("x", 10, 8)]) | D.FeatureSet([D.SparseFeature("y", 10, 16)])
  with pytest.raises(ValueError, match="embedding_dim"):
    D.ModelConfig.from_features(mixed)


@pytest.mark.parametrize("rank", [None, 5])
def test_cross_network_is_the_dcn_v2_recurrence(rank):
  """`xl <- x0 * ((xl U) V + b) + xl` (low rank) or `x0 * (W xl + b) + xl` written out with plain matrix products
  (`recml/examples/dlrm_experiment.py:154-177`), values and gradients."""
  import torch
  from recml_b200.layers import dcn
  torch.manual_seed(0)
  net = dcn.CrossNetwork(12, 3, rank)
  with torch.no_grad():
    for b in net.b:
      b.normal_()
  x0 = torch.randn(7, 12, requires_grad=True)
  x1 = x0.detach().clone().requires_grad_()
  out = net(x0)
  xl = x1
  for i in range(3):
    h = xl @ net.u[i].t() @ net.v[i].t() if rank else xl @ net.v[i].t()
    xl = x1 * (h + net.b[i]) + xl
  torch.testing.assert_close(out, xl, rtol=1e-5, atol=1e-5)
  g = torch.randn_like(out)
  out.backward(g)
  grads = [p.grad.clone() for p in net.parameters()]
  net.zero_grad()
  xl.backward(g)
  torch.testing.assert_close(x0.grad, x1.grad, rtol=1e-4, atol=1e-5)
  for a, p in zip(grads, net.parameters()):
    torch.testing.assert_close(a, p.grad, rtol=1e-4, atol=1e-5)


def test_dlrm_forward_equals_a_plain_torch_restatement():
  """The whole DLRM-DCNv2 forward on one CPU rank against the model written with `embedding_bag`, `linear`, `relu`
  and the cross recurrence, using the module's own weights and tables (the architecture of
  `recml/examples/dlrm_experiment.py:100-236`: bottom MLP, one pooled embedding per feature, concat, cross, top)."""
  import torch
  import torch.nn.functional as F
  from recml_b200 import embedding as emb
  from recml_b200.models import dlrm
  torch.manual_seed(0)
  rng = np.random.default_rng(0)
  vocab, bags, B = [50, 7, 300], [3, 1, 4], 9
  m = dlrm.DLRMDCNv2(vocab_sizes=vocab, embedding_dim=8, num_dense=5, bottom_mlp_dims=(16, 8), top_mlp_dims=(12, 1),
                     num_cross_layers=2, cross_rank=4, bag_sizes=bags, device="cpu", backend="collective", init_scale=0.1)
  with torch.no_grad():
    for p in m.parameters():
      if p.ndim == 1:
        p.normal_(std=0.1)                      # biases are zero at initialisation
  dense_x = torch.randn(B, 5)
  ids = {f"cat_{i}": [rng.integers(0, v, b).tolist() for _ in range(B)] for i, (v, b) in enumerate(zip(vocab, bags))}
  got = m(dense_x, emb.KeyedJagged.from_lists(ids))

  def mlp(x, net):
    for w, b, act in zip(net.weights, net.biases, net.relu_flags):
      x = F.linear(x, w, b)
      x = F.relu(x) if act else x
    return x
  parts = [mlp(dense_x, m.bottom)]
  for name in ids:
    flat = torch.tensor([i for bag in ids[name] for i in bag])
    offs = torch.tensor(np.cumsum([0] + [len(bag) for bag in ids[name][:-1]]))
    parts.append(F.embedding_bag(flat, m.embedding.gather_table(name), offs, mode="sum"))
  x0 = xl = torch.cat(parts, dim=1)
  for u, v, b in zip(m.cross.u, m.cross.v, m.cross.b):
    xl = x0 * (xl @ u.t() @ v.t() + b) + xl
  want = mlp(xl, m.top).reshape(-1)
  torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-5)
