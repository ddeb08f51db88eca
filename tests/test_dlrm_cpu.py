"""DLRM experiment pieces that need no GPU."""
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
