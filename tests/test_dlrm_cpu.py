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
